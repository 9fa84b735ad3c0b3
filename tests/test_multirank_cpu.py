"""world_size-2 host logic on CPU (gloo): rank -> TP-rank mapping, the address
exchange, the push plan and its ordering against the barrier.  The ranks'
'device memory' is a /dev/shm file every rank maps, and the records are executed
by the oracle's C loop, so no GPU is needed."""

import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent('''
    import os, sys, mmap
    import numpy as np
    import torch, torch.distributed as dist
    sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import read_full_tensors, run_records_on_host, tiny_dense_config
    from modelexpress_b200 import layout, reshard, synth
    from modelexpress_b200.safetensors_index import checkpoint_index
    from oracle import ref_port as R

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    work = os.environ["MXB_TEST_DIR"]
    cfg = tiny_dense_config()
    ckpt = os.path.join(work, "ckpt")
    if rank == 0:
        synth.write_checkpoint(ckpt, synth.dense_tensors(cfg), cfg.seed, 1)
    dist.barrier()
    full = read_full_tensors(ckpt)
    idx = checkpoint_index(ckpt)
    index = {n: {"shape": i["shape"], "dtype": i["dtype"]} for n, i in idx.items()}
    LOGICAL = 8                      # 8 trainer ranks and 8 inference ranks over `world` processes
    mine = [r for r in range(LOGICAL) if r % world == rank]
    sa = reshard.shard_arena(index, LOGICAL)
    pa = reshard.param_arena(layout.plan_checkpoint(index, 0, LOGICAL))

    def shared(name, nbytes, create):
        path = os.path.join(work, name)
        if create:
            with open(path, "wb") as f:
                f.truncate(nbytes)
        f = open(path, "r+b")
        return np.frombuffer(mmap.mmap(f.fileno(), nbytes), dtype=np.uint8)

    # every process owns one "parameter arena" file; peers map it (the IPC stand-in)
    own = shared(f"params{rank}", pa.total * len(mine), True)
    dist.barrier()
    maps = [own if r == rank else shared(f"params{r}", pa.total * len(mine), False) for r in range(world)]
    bases = [m.ctypes.data for m in maps]
    # exchange something real: every rank announces its logical ranks
    hosted = [None] * world
    dist.all_gather_object(hosted, mine)
    assert sorted(sum(hosted, [])) == list(range(LOGICAL))
    param_bases = [bases[t % world] + (t // world) * pa.total for t in range(LOGICAL)]
    pieces = R.fsdp_shards(full, LOGICAL)
    moved = 0
    for j, s in enumerate(mine):
        arena = np.zeros(sa.total, dtype=np.uint8)
        for n, piece in pieces[s].items():
            b = piece.view(np.uint8)
            arena[sa.offsets[n]: sa.offsets[n] + b.size] = b
        recs = reshard.plan_reshard(index, LOGICAL, LOGICAL, s, arena.ctypes.data, param_bases,
                                    shards=sa, params=pa)
        moved += reshard.reshard_bytes(recs)
        run_records_on_host(recs)        # pushes into local AND peer arenas
    for m in maps:
        if hasattr(m, "flush"):
            pass
    dist.barrier()                        # all pushes landed before anyone reads
    shapes = {n: a.shape for n, a in full.items()}
    for j, t in enumerate(mine):
        want = R.regather_and_reslice(pieces, shapes, t, LOGICAL)
        for n, a in want.items():
            o = j * pa.total + pa.offsets[n]
            got = own[o: o + a.nbytes].view(a.dtype).reshape(a.shape)
            assert np.array_equal(got, a), (rank, t, n)
    tot = torch.tensor([moved], dtype=torch.int64)
    dist.all_reduce(tot)
    expect = sum(a.nbytes for a in R.load_and_shard(full, 0, LOGICAL).values()) * LOGICAL
    assert int(tot.item()) == expect, (int(tot.item()), expect)
    dist.barrier()
    dist.destroy_process_group()
    print("rank", rank, "ok")
''')


@pytest.mark.parametrize("world", [2])
def test_reshard_push_plan_two_ranks_gloo(tmp_path, world):
    script = tmp_path / "worker.py"
    script.write_text(f"ROOT = {ROOT!r}\n" + WORKER)
    env = dict(os.environ, MXB_TEST_DIR=str(tmp_path), MASTER_ADDR="127.0.0.1")
    port = 29600 + (os.getpid() % 300)
    proc = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
         "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
        env=env, capture_output=True, text=True, timeout=240)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert proc.stdout.count("ok") == world


def test_bench_rank_mapping_and_reference_arm_ranks():
    """bench.py: TP rank = rank mod 8; under torchrun only rank 0 of the
    reference arm works, the others return at once."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert bench.TP == 8
    os.environ["RANK"] = "3"
    try:
        class A:
            gpus, steps, warmup = 4, 1, 0
        assert bench.bench_reference(A()) is None  # rank != 0: no work, no output
    finally:
        os.environ.pop("RANK")
