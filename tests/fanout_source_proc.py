"""Child process of tests/test_gpu_fanout_strategy.py: a serving peer.

    python tests/fanout_source_proc.py <rendezvous dir> <source id> <seed> <mode>

Builds the seeded tensors on cuda:0, publishes the manifest, prints ``ready``, then
(mode ``serve``, or ``serve256`` with the default chunk and piece sizes) answers one request
and prints ``served``, or (mode ``silent``) answers nothing.  Stays alive, keeping its memory mapped for the peer, until a line arrives on
stdin."""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def seeded_tensors(seed: int, device: str = "cuda"):
    import torch

    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    shapes = {"embed.weight": (1000, 256), "layers.0.qkv.weight": (768, 256), "layers.0.qkv.bias": (768,),
              "layers.0.down.weight": (256, 1024), "norm.weight": (256,), "odd.bytes": (4099,)}
    out = {}
    for name, shape in shapes.items():
        if name == "odd.bytes":
            out[name] = torch.randint(0, 256, shape, generator=g, dtype=torch.uint8).to(device)
        else:
            out[name] = torch.randn(shape, generator=g).to(torch.bfloat16).to(device)
    return out


def main():
    import torch

    from modelexpress_b200.fanout import FanoutSource

    rendezvous, source_id, seed, mode = sys.argv[1], sys.argv[2], int(sys.argv[3]), sys.argv[4]
    torch.cuda.set_device(0)
    tensors = seeded_tensors(seed)
    if mode == "serve256":      # the defaults of a one-hop push: 256 KiB chunks of one 256 KiB piece
        src = FanoutSource(tensors, rendezvous, source_id)
        assert src.piece_bytes == 256 << 10
    else:
        src = FanoutSource(tensors, rendezvous, source_id, chunk_bytes=64 << 10)
    src.publish()
    print("ready", flush=True)
    if mode in ("serve", "serve256"):
        n = src.serve(timeout_s=60.0, max_requests=1)
        print(f"served {n}", flush=True)
    sys.stdin.readline()
    src.close()


if __name__ == "__main__":
    main()
