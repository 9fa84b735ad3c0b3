"""The device arena on CUDA virtual memory management: lifecycle as the reference's VmmArena
(vmm/arena.py:155-350), torch routed into it (vmm/hook.py:164-200), and the crossing of a
process boundary that replaces one IPC handle per allocation."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest

from make_golden import golden_bytes

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_lifecycle_and_kernels_on_arena_memory():
    import torch

    from modelexpress_b200._lib import MxbError
    from modelexpress_b200.arena import Arena
    from modelexpress_b200.runtime import Context

    ctx = Context([0])
    arena = Arena(0, 1 << 30)
    gran = arena.blocks() == [] and arena.total_bytes
    assert gran >= 1 << 30 and arena.used_bytes == 0 and arena.live_allocation_count == 0
    p1 = arena.malloc(1000)                     # rounded up to the granularity
    p2 = arena.malloc(5 << 20)
    blocks = arena.blocks()
    assert [o for o, _s in blocks] == [p1 - arena.base, p2 - arena.base]
    g = blocks[0][1]
    assert g >= 2 << 20 and g & (g - 1) == 0 and blocks[1][1] % g == 0 and blocks[1][1] >= 5 << 20
    assert arena.registered_range() == (arena.base, blocks[0][1] + blocks[1][1])
    assert arena.contains(p2, 5 << 20) and not arena.contains(arena.base + arena.used_bytes)
    # the scatter kernel writes and reads arena memory like any other device memory
    src = torch.from_numpy(golden_bytes(7, 5 << 20)).cuda()
    back = torch.zeros(5 << 20, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    ctx.scatter([(src.data_ptr(), p2, 1, 5 << 20, 5 << 20, 5 << 20)], 0)
    ctx.scatter([(p2 + 4096, back.data_ptr() + 4096, 512, 1024, 8192, 8192)], 0)
    want = np.zeros(5 << 20, dtype=np.uint8)
    ref = golden_bytes(7, 5 << 20)
    for r in range(512):
        want[4096 + r * 8192: 4096 + r * 8192 + 1024] = ref[4096 + r * 8192: 4096 + r * 8192 + 1024]
    assert np.array_equal(back.cpu().numpy(), want)
    rec = ctx.digest([(p2, 5 << 20)], 1, 0)[0]
    from oracle import ref_port as R
    assert format(rec.safe_checksum, "08x") == R.safe_checksum(ref)
    arena.free(p1)
    assert arena.live_allocation_count == 1
    p3 = arena.malloc(1)
    assert p3 > p2                                # offsets are never reused
    with pytest.raises(MxbError):
        arena.free(p1)                            # already gone
    with pytest.raises(MxbError):
        arena.malloc(2 << 30)                     # past the reserved range
    with pytest.raises(ValueError):
        arena.malloc(0)
    arena.close()
    arena.close()                                 # idempotent
    ctx.close()


def test_torch_allocates_inside_use_arena():
    import torch

    from modelexpress_b200.arena import Arena, use_arena

    arena = Arena(0, 4 << 30)
    outside = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    with use_arena(arena):
        w = torch.empty(3000, 1024, dtype=torch.bfloat16, device="cuda")
        v = torch.zeros(17, dtype=torch.float32, device="cuda")
    after = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    assert arena.contains(w.data_ptr(), w.numel() * 2) and arena.contains(v.data_ptr(), 68)
    assert not arena.contains(outside.data_ptr()) and not arena.contains(after.data_ptr())
    w.normal_()
    assert torch.isfinite(w.float()).all() and float(v.sum()) == 0.0
    assert arena.mapped_bytes >= w.numel() * 2
    # a second arena gets its own torch pool: nothing of the first arena's cache leaks into it
    second = Arena(0, 4 << 30)
    del v
    with use_arena(second):
        v2 = torch.zeros(17, dtype=torch.float32, device="cuda")
    assert second.contains(v2.data_ptr(), 68) and not arena.contains(v2.data_ptr())
    del w, v2
    torch.cuda.synchronize()
    second.close()
    arena.close()


def _peer(tmp_path, peer_dev, my_dev):
    import torch

    from modelexpress_b200 import digest
    from modelexpress_b200.arena import fetch_arena
    from modelexpress_b200.runtime import Context

    sock, report = str(tmp_path / "arena.sock"), str(tmp_path / "report.json")
    p = subprocess.Popen([sys.executable, os.path.join(HERE, "arena_peer_proc.py"), sock, report, "5", str(peer_dev)],
                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        assert p.stdout.readline().strip() == "ready"
        with open(report) as f:
            rep = json.load(f)
        torch.cuda.set_device(my_dev)
        ctx = Context([my_dev])
        peer = fetch_arena(sock, my_dev)
        assert [list(b) for b in peer.blocks()] == [list(b) for b in rep["blocks"]]
        a_off, a_n, a_sum = rep["a"]
        # read the peer's first tensor through the one mapping: digest in place, then copy out
        rec = ctx.digest([(peer.base + a_off, a_n)], 1, my_dev)[0]
        assert format(rec.safe_checksum, "08x") == a_sum
        mine = torch.zeros(a_n, dtype=torch.uint8, device=f"cuda:{my_dev}")
        torch.cuda.synchronize(my_dev)
        ctx.scatter([(peer.base + a_off, mine.data_ptr(), 1, a_n, a_n, a_n)], my_dev)
        assert digest.safe_checksum(mine) == a_sum
        # and write into its second tensor
        b_off, b_n = rep["b"]
        payload = torch.from_numpy(golden_bytes(9, b_n)).to(f"cuda:{my_dev}")
        torch.cuda.synchronize(my_dev)
        ctx.scatter([(payload.data_ptr(), peer.base + b_off, 1, b_n, b_n, b_n)], my_dev)
        ctx.sync(my_dev)
        p.stdin.write("check\n")
        p.stdin.flush()
        assert p.stdout.readline().strip() == "b " + digest.safe_checksum(payload)
        peer.close()
        ctx.close()
        p.stdin.write("bye\n")
        p.stdin.flush()
        p.wait(timeout=30)
    finally:
        if p.poll() is None:
            p.kill()


def test_another_process_maps_the_arena_same_gpu(tmp_path):
    _peer(tmp_path, 0, 0)


def test_another_process_maps_the_arena_across_gpus(tmp_path):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _peer(tmp_path, 1, 0)
