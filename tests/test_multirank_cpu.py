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


REFIT_WORKER = textwrap.dedent('''
    import os, sys, mmap
    import numpy as np
    import torch, torch.distributed as dist
    sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests"))
    import hooked_model as H
    from helpers import run_records_on_host
    from modelexpress_b200.geometry import capture_geometry
    from modelexpress_b200.planner import plan_transfer_2d
    from modelexpress_b200.refit import (PublishedShard, PublishedTensor, build_sources,
                                         decode_shard_table, encode_shard_table, merge_shard_tables)

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    work = os.environ["MXB_TEST_DIR"]
    H.TP, H.RANK = world, rank          # this process is inference TP rank `rank` ...
    man = H.manifest()
    g = torch.Generator().manual_seed(11)
    full = {n: torch.randn(s, generator=g) for n, _d, s in man}   # same in every process

    # ... and trainer rank `rank`: it owns row block `rank` of every tensor, laid out
    # back to back in a file the other processes map (the stand-in for a CUDA IPC mapping)
    def block(t, r):
        rows = t.shape[0]
        lo, hi = r * rows // world, (r + 1) * rows // world
        return lo, t[lo:hi].contiguous()

    total = sum(block(t, rank)[1].numel() * 4 for t in full.values())
    path = os.path.join(work, f"trainer{rank}")
    with open(path, "wb") as f:
        f.truncate(total)
    fh = open(path, "r+b")
    mine = np.frombuffer(mmap.mmap(fh.fileno(), total), dtype=np.uint8)
    table, at = [], 0
    for n, t in full.items():
        lo, piece = block(t, rank)
        raw = piece.numpy().view(np.uint8).reshape(-1)
        mine[at: at + raw.size] = raw
        table.append(PublishedTensor(n, "torch.float32", 4, tuple(t.shape), [PublishedShard(
            f"trainer{rank}", 0, mine.ctypes.data + at, (lo,) + (0,) * (t.dim() - 1), tuple(piece.shape))]))
        at += raw.size
    dist.barrier()                       # every trainer file is written

    # rendezvous: wire blobs and each publisher's base address (an IPC handle + offset in real life)
    blobs, bases = [None] * world, [None] * world
    dist.all_gather_object(blobs, encode_shard_table(table))
    dist.all_gather_object(bases, (total, mine.ctypes.data))
    local = {}
    for r, (nbytes, _addr) in enumerate(bases):
        if r == rank:
            local[f"trainer{r}"] = mine.ctypes.data
        else:
            f2 = open(os.path.join(work, f"trainer{r}"), "r+b")
            m = np.frombuffer(mmap.mmap(f2.fileno(), nbytes), dtype=np.uint8)
            local[f"trainer{r}"] = (m, m.ctypes.data)
    def map_address(s):
        r = int(s.agent_name[len("trainer"):])
        here = local[s.agent_name]
        here = here if isinstance(here, int) else here[1]
        return here + (s.addr - bases[r][1])
    merged = merge_shard_tables([decode_shard_table(b) for b in blobs])
    assert all(len(t.shards) == world for t in merged)
    sources = build_sources(merged, map_address)

    model = H.HookedModel()
    cap = capture_geometry(model, man)
    assert cap.unsupported == []
    params = dict(model.named_parameters())
    recs, unsupported, converts = plan_transfer_2d(cap.copies, sources, lambda n: params[n].data_ptr())
    assert not unsupported and not converts
    run_records_on_host(recs)            # reads local and peer trainer memory
    truth = H.HookedModel()
    truth.load_weights(full.items())
    for (n, a), (_n, b) in zip(model.state_dict().items(), truth.state_dict().items()):
        assert torch.equal(a, b), (rank, n)
    # bytes read from the peer: everything this rank needs that the other trainer owns
    peer = sum(int(r[2]) * int(r[3]) for r in recs.tolist()
               if not (mine.ctypes.data <= int(r[0]) < mine.ctypes.data + total))
    tot = torch.tensor([peer], dtype=torch.int64)
    dist.all_reduce(tot)
    assert int(tot.item()) > 0
    dist.barrier()
    dist.destroy_process_group()
    print("rank", rank, "ok")
''')


@pytest.mark.parametrize("world", [2])
def test_refit_cycle_two_ranks_gloo(tmp_path, world):
    """Two processes, each a trainer rank and an inference TP rank: shard tables
    travel as wire blobs over gloo, are merged, mapped to local addresses and
    planned from the captured loader; the CPU scatter then assembles every
    parameter from local and peer trainer memory."""
    script = tmp_path / "refit_worker.py"
    script.write_text(f"ROOT = {ROOT!r}\n" + REFIT_WORKER)
    env = dict(os.environ, MXB_TEST_DIR=str(tmp_path), MASTER_ADDR="127.0.0.1")
    port = 29300 + (os.getpid() % 250)
    proc = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
         "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
        env=env, capture_output=True, text=True, timeout=240)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert proc.stdout.count("ok") == world


FANOUT_WORKER = textwrap.dedent('''
    import os, sys, mmap, ctypes
    import numpy as np
    import torch, torch.distributed as dist
    sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests"))
    from modelexpress_b200.fanout import (ManifestMismatchError, TensorDescriptor, match_manifests,
                                          plan_pieces, topology)

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    work = os.environ["MXB_TEST_DIR"]
    sizes = [3 << 20, 4096 + 16, 100, 333 * 16, 1 << 20, 52, 700_000]
    names = [f"t{i}" for i in range(len(sizes))]
    CHUNK = 256 << 10

    def shared(name, nbytes, create):
        path = os.path.join(work, name)
        if create:
            with open(path, "wb") as f:
                f.truncate(nbytes)
        f = open(path, "r+b")
        return np.frombuffer(mmap.mmap(f.fileno(), nbytes), dtype=np.uint8)

    offs, pos = [], 0
    for n in sizes:
        offs.append(pos)
        pos = (pos + n + 255) // 256 * 256
    pieces, chunk_pieces = plan_pieces(sizes, CHUNK)
    # every rank owns a payload arena and its arrival counters; peers map both (the IPC stand-in)
    own = shared(f"arena{rank}", pos, True)
    ctr = shared(f"ctr{rank}", 4 * len(chunk_pieces), True).view(np.uint32)
    if rank == 0:
        rng = np.random.default_rng(3)
        own[:] = rng.integers(0, 256, pos, dtype=np.uint8)
    dist.barrier()
    arenas = [own if r == rank else shared(f"arena{r}", pos, False) for r in range(world)]
    ctrs = [ctr if r == rank else shared(f"ctr{r}", 4 * len(chunk_pieces), False).view(np.uint32)
            for r in range(world)]
    # the manifests travel between the ranks; every target matches the root's against its own
    mine = [TensorDescriptor(n, int(arenas[rank].ctypes.data) + o, s, rank, "torch.uint8")
            for n, o, s in zip(names, offs, sizes)]
    everyone = [None] * world
    dist.all_gather_object(everyone, [(d.name, d.size, d.dtype) for d in mine])
    root_rows = [TensorDescriptor(n, 0, s, 0, dt) for n, s, dt in everyone[0]]
    matched = match_manifests(root_rows, mine)
    assert [m[0] for m in matched] == names and [m[3] for m in matched] == sizes
    try:
        match_manifests(root_rows[:-1], mine)
        raise SystemExit("a missing tensor went unnoticed")
    except ManifestMismatchError:
        pass
    try:
        match_manifests([TensorDescriptor("t0", 0, sizes[0] + 2, 0, "torch.uint8")] + root_rows[1:], mine)
        raise SystemExit("a size mismatch went unnoticed")
    except ManifestMismatchError:
        pass
    # the piece plan depends on sizes only: every rank cut the same pieces
    plans = [None] * world
    dist.all_gather_object(plans, (pieces, chunk_pieces))
    assert all(p == plans[0] for p in plans)
    assert sum(p[2] for p in pieces) == sum(sizes) and max(p[2] for p in pieces) <= 65536
    assert all(p[1] % 16 == 0 for p in pieces) and sum(chunk_pieces) == len(pieces)
    # one broadcast down the chain, executed piece by piece on the host the way a node's kernel
    # does it: wait for the chunk's counter (not the root), store to the child, raise its counter
    children = topology("chain", world, 0)
    run_index = 1
    for rng_i, off, nbytes, chunk in pieces:
        if rank != 0:
            import time
            t0 = time.time()
            while int(ctrs[rank][chunk]) < run_index * chunk_pieces[chunk]:
                assert time.time() - t0 < 60, "chunk never arrived"
                time.sleep(0.0002)
        for c in children[rank]:
            a = offs[rng_i] + off
            arenas[c][a: a + nbytes] = arenas[rank][a: a + nbytes]
        # all of a chunk's pieces stored before its counter moves: here one piece at a time
        for c in children[rank]:
            ctrs[c][chunk] += 1
    dist.barrier()
    if rank != 0:
        for o, s in zip(offs, sizes):
            assert np.array_equal(arenas[rank][o: o + s], arenas[0][o: o + s])
        assert [int(x) for x in ctrs[rank]] == chunk_pieces
    dist.barrier()
    dist.destroy_process_group()
    print("rank", rank, "ok")
''')


def test_fanout_host_logic_two_ranks_gloo(tmp_path):
    """Topology, manifest exchange and matching, the piece / chunk plan of the library
    and the arrival-counter bookkeeping of one chain broadcast, two processes over gloo
    with /dev/shm-style shared files standing in for peer-mapped GPU memory."""
    script = tmp_path / "fanout_worker.py"
    script.write_text(f"ROOT = {ROOT!r}\n" + FANOUT_WORKER)
    env = dict(os.environ, MXB_TEST_DIR=str(tmp_path), MASTER_ADDR="127.0.0.1")
    port = 29300 + (os.getpid() % 300)
    proc = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
        env=env, capture_output=True, text=True, timeout=240)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert proc.stdout.count("ok") == 2
