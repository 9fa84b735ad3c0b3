"""Child process of tests/test_gpu_arena.py: owns an arena and serves it.

    python tests/arena_peer_proc.py <socket path> <report path> <seed> <device>

Allocates two tensors through torch inside ``use_arena`` (so they live in the arena), fills
them from the seed, serves the arena on the socket, writes a report (offsets, sizes, digests),
prints ``ready``.  After a line on stdin it prints the checksum of the second tensor again (the
parent may have written into it) and exits."""

import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch

    from modelexpress_b200 import digest
    from modelexpress_b200.arena import Arena, ArenaServer, use_arena

    sock, report, seed, dev = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4])
    torch.cuda.set_device(dev)
    arena = Arena(dev, 8 << 30)
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    with use_arena(arena):
        a = torch.empty(5 << 20, dtype=torch.uint8, device=f"cuda:{dev}")
        b = torch.empty(3 << 20, dtype=torch.uint8, device=f"cuda:{dev}")
    a.copy_(torch.randint(0, 256, (a.numel(),), generator=g, dtype=torch.uint8))
    b.zero_()
    torch.cuda.synchronize(dev)
    assert arena.contains(a.data_ptr(), a.numel()) and arena.contains(b.data_ptr(), b.numel())
    server = ArenaServer(arena, sock)
    with open(report, "w") as f:
        json.dump({"a": [a.data_ptr() - arena.base, a.numel(), digest.safe_checksum(a)],
                   "b": [b.data_ptr() - arena.base, b.numel()], "blocks": arena.blocks()}, f)
    print("ready", flush=True)
    sys.stdin.readline()
    torch.cuda.synchronize(dev)
    print(f"b {digest.safe_checksum(b)}", flush=True)
    server.close()
    del a, b
    sys.stdin.readline()


if __name__ == "__main__":
    main()
