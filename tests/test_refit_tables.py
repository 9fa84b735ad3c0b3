"""Shard-table helpers of the refit receiver (no GPU): replica de-duplication,
cross-rank fan-in, consistency checks and address mapping — the behaviours the
reference pins in tests/test_reshard_refit_replica_merge.py:90-200."""

import numpy as np
import pytest
import torch

from modelexpress_b200.planner import CopySpec, expand_records, plan_transfer_2d
from modelexpress_b200.refit import (PublishedShard, PublishedTensor, build_sources,
                                     merge_shard_tables)

EL = 2


def _replicas(n, shards_per_rank=2):
    return [[PublishedTensor("weight", "torch.bfloat16", EL, (8, 4), [
        PublishedShard(f"dp{dp}", dp, 1000 * (dp + 1) + 10 * i, (4 * i, 0), (4, 4))
        for i in range(shards_per_rank)])] for dp in range(n)]


def _fan_in(ranks=4):
    return [[PublishedTensor("weight", "torch.bfloat16", EL, (16, 4), [
        PublishedShard(f"r{r}", r, 1000 * (r + 1), (4 * r, 0), (4, 4))])] for r in range(ranks)]


def test_replicas_collapse_to_the_first_publisher():
    (t,) = merge_shard_tables(_replicas(8))
    assert [(s.agent_name, s.shard_offset) for s in t.shards] == [("dp0", (0, 0)), ("dp0", (4, 0))]


def test_dedup_removes_reads_not_only_offers():
    copy = CopySpec("weight", (), "p", 0, (8, 4), (4, 1), torch.bfloat16)
    for tables, n_reads in ((_replicas(1), 2), (_replicas(8), 2)):
        sources = build_sources(merge_shard_tables(tables))
        table, unsupported, converts = plan_transfer_2d([copy], sources, lambda n: 1 << 20)
        assert not unsupported and not converts
        runs = expand_records(table)
        assert len(runs) == n_reads and sum(r[2] for r in runs) == 8 * 4 * EL


def test_distinct_geometry_is_kept_for_every_rank():
    (t,) = merge_shard_tables(_fan_in(4))
    assert [s.agent_name for s in t.shards] == ["r0", "r1", "r2", "r3"]
    # replicated fan-in: every region once, from its first publisher
    (t,) = merge_shard_tables(_fan_in(4) + _fan_in(4))
    assert [s.shard_offset for s in t.shards] == [(0, 0), (4, 0), (8, 0), (12, 0)]


def test_inconsistent_shape_or_dtype_raises():
    a = [PublishedTensor("w", "torch.bfloat16", 2, (8, 4), [])]
    with pytest.raises(ValueError, match="inconsistent"):
        merge_shard_tables([a, [PublishedTensor("w", "torch.bfloat16", 2, (4, 4), [])]])
    with pytest.raises(ValueError, match="inconsistent"):
        merge_shard_tables([a, [PublishedTensor("w", "torch.float16", 2, (8, 4), [])]])


def test_names_are_independent_and_addresses_can_be_mapped():
    tables = [[PublishedTensor("a", "torch.bfloat16", 2, (4, 4), [PublishedShard("r0", 0, 100, (0, 0), (4, 4), "d0")]),
               PublishedTensor("b", "torch.float32", 4, (2,), [PublishedShard("r0", 0, 200, (0,), (2,))])]]
    merged = merge_shard_tables(tables)
    assert [t.name for t in merged] == ["a", "b"]
    sources = build_sources(merged, map_address=lambda s: (1 << 30) + s.addr)
    assert sources["a"].shards[0].addr == (1 << 30) + 100 and sources["a"].shards[0].digest == "d0"
    assert sources["a"].dtype == torch.bfloat16 and sources["b"].dtype == torch.float32
    assert sources["b"].global_shape == (2,) and sources["b"].elsize == 4
    assert np.asarray(sources["a"].shards[0].shard_offset).tolist() == [0, 0]


def test_shard_table_wire_blob_is_the_references():
    """``shard_table.json`` holds the blob the reference's encode_shard_table wrote
    for this table; ours must be byte-identical and decode back to the same."""
    import json
    import os

    from modelexpress_b200.refit import decode_shard_table, encode_shard_table

    with open(os.path.join(os.path.dirname(__file__), "golden", "shard_table.json")) as f:
        want = json.load(f)["blob"].encode("utf-8")
    table = [
        PublishedTensor("model.layers.0.self_attn.q_proj.weight", "torch.bfloat16", 2, (4096, 4096), [
            PublishedShard("trainer-0", 0, 140000000000000, (0, 0), (512, 4096), "00112233445566778899aabbccddeeff"),
            PublishedShard("trainer-1", 1, 140000004194304, (512, 0), (512, 4096), None)]),
        PublishedTensor("model.norm.weight", "torch.float32", 4, (4096,), [
            PublishedShard("trainer-0", 0, 140000008388608, (0,), (4096,), "ffeeddccbbaa99887766554433221100")]),
    ]
    assert encode_shard_table(table) == want
    back = decode_shard_table(want)
    assert back == table and back[0].shards[1].digest is None
    assert b'"digest": null' not in want
    with pytest.raises(ValueError, match="schema"):
        decode_shard_table(want.replace(b"shard_table.v1", b"shard_table.v9"))


def test_coverage_gate_is_opt_in_and_names_what_is_missed(monkeypatch):
    """receiver.py:746-755: off by default (partial refits are a feature); with the
    switch on, a plan below the floor raises IncompleteRefit, not a planning error."""
    from modelexpress_b200.refit import IncompleteRefit, check_coverage

    monkeypatch.delenv("MXB_RESHARD_REQUIRE_FULL_COVERAGE", raising=False)
    monkeypatch.delenv("MX_RESHARD_REQUIRE_FULL_COVERAGE", raising=False)
    check_coverage(0.5, 50, 100, ["a", "b"], 4)                      # off: nothing happens
    monkeypatch.setenv("MXB_RESHARD_REQUIRE_FULL_COVERAGE", "true")
    check_coverage(0.9999, 9999, 10000, [], 4)                       # above the default floor 0.995
    with pytest.raises(IncompleteRefit, match=r"50.00%.*2 of 4 params.*\['a', 'b'\]"):
        check_coverage(0.5, 50, 100, ["b", "a"], 4)
    assert not issubclass(IncompleteRefit, ValueError) and issubclass(IncompleteRefit, RuntimeError)
    monkeypatch.setenv("MXB_RESHARD_COVERAGE_FLOOR", "0.4")
    check_coverage(0.5, 50, 100, ["a"], 4)                           # floor lowered per model
    # the reference's own variable names are honoured where ours are unset
    monkeypatch.delenv("MXB_RESHARD_REQUIRE_FULL_COVERAGE")
    monkeypatch.delenv("MXB_RESHARD_COVERAGE_FLOOR")
    monkeypatch.setenv("MX_RESHARD_REQUIRE_FULL_COVERAGE", "1")
    with pytest.raises(IncompleteRefit):
        check_coverage(0.9, 90, 100, ["a"], 4)


def test_throughput_ceiling_refuses_an_impossible_step(monkeypatch, caplog):
    """receiver.py:1045-1106 with fabricated timings: off unless configured, a
    non-finite ceiling disables it, a rate above it aborts after logging the record."""
    import logging

    from modelexpress_b200.refit import check_throughput_ceiling

    monkeypatch.delenv("MXB_RESHARD_MAX_GBPS", raising=False)
    monkeypatch.delenv("MX_RESHARD_MAX_GBPS", raising=False)
    check_throughput_ceiling(1, 40_610_000_000, 0.84)                # off
    for off in ("nan", "inf", "0", "-5", "junk"):
        monkeypatch.setenv("MXB_RESHARD_MAX_GBPS", off)
        check_throughput_ceiling(1, 40_610_000_000, 0.0001)
    monkeypatch.setenv("MXB_RESHARD_MAX_GBPS", "191")
    check_throughput_ceiling(2, 40_610_000_000, 2.0)                 # 162 Gbps: fine
    check_throughput_ceiling(2, 0, 0.001)                            # nothing moved: nothing to judge
    with caplog.at_level(logging.WARNING, logger="modelexpress_b200.refit"):
        with pytest.raises(RuntimeError, match=r"implied 386\.8 Gbps against a per-rank ceiling of 191\.0"):
            check_throughput_ceiling(3, 40_610_000_000, 0.84)        # the reference's own anecdote
    assert "MX_REFIT_IMPOSSIBLE_THROUGHPUT" in caplog.text and '"step": 3' in caplog.text
