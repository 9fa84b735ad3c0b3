"""The oracle's restatement of the strided, casting copy a pull ends with, pinned to the call
the reference makes (`dst.copy_(staged)`, refit/reshard/receiver.py:964-971) on host tensors."""

import itertools

import numpy as np
import torch

from oracle import ref_port as R


def test_bf16_rounding_matches_torch():
    rng = np.random.default_rng(3)
    bits = rng.integers(0, 1 << 32, size=200000, dtype=np.uint64).astype(np.uint32)
    x = bits.view(np.float32)
    x = x[~np.isnan(x)]
    x = np.concatenate([x, np.array([0.0, -0.0, np.inf, -np.inf, 1e-40, -1e-45, 3.3895313892515355e38,
                                      1.00390625, 1.01171875], dtype=np.float32)])
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(R.f32_to_bf16_bits(x), want)
    back = torch.from_numpy(want.view(np.int16)).view(torch.bfloat16).float().numpy()
    assert np.array_equal(R.bf16_bits_to_f32(want).view(np.uint32), back.view(np.uint32))


def test_box_convert_matches_torch_strided_copy():
    rng = np.random.default_rng(4)
    shape = (3, 4, 5, 6)
    src = rng.integers(0, 1 << 15, size=int(np.prod(shape)), dtype=np.int16)
    for perm in itertools.permutations(range(4)):
        out_shape = [shape[p] for p in perm]
        out_strides = [int(np.prod(out_shape[k + 1:])) for k in range(4)]
        strides = [0] * 4
        for k, p in enumerate(perm):
            strides[p] = out_strides[k]
        got = np.zeros(src.size + 7, dtype=np.int16)
        R.box_convert(src, shape, strides, got, dst_offset=5)
        want = torch.zeros(src.size + 7, dtype=torch.int16)
        torch.as_strided(want, shape, strides, 5).copy_(torch.from_numpy(src).reshape(shape))
        assert np.array_equal(got, want.numpy()), perm
    # a column window of a wider parameter, narrowed on the way
    m, n = 7, 9
    x = rng.standard_normal(m * n).astype(np.float32)
    got = np.zeros(n * (m + 3), dtype=np.uint16)
    R.box_convert(x, (m, n), (1, m + 3), got, dst_offset=2, cast=R.f32_to_bf16_bits)
    want = torch.zeros(n * (m + 3), dtype=torch.bfloat16)
    torch.as_strided(want, (m, n), (1, m + 3), 2).copy_(torch.from_numpy(x).reshape(m, n))
    assert np.array_equal(got, want.view(torch.int16).numpy().view(np.uint16))
    R.box_convert(np.zeros(0, dtype=np.int16), (0, 4), (4, 1), got)   # empty: nothing written


def _run_boxes_on_host(boxes):
    """The convert kernel's definition executed with numpy over raw addresses (fp32 -> bf16 and
    bf16 -> fp32 boxes of rank 2 with source strides), the checker for `planner.direct_cast`."""
    import ctypes

    for src, dst, extents, dst_strides, sk, dk, _eb, src_strides in boxes:
        rows, cols = extents
        assert src_strides[1] == 1 and dst_strides[1] == 1
        s_t, d_t = {"f32": ctypes.c_float, "bf16": ctypes.c_uint16}[sk], {"f32": ctypes.c_float, "bf16": ctypes.c_uint16}[dk]
        for r in range(rows):
            row = np.ctypeslib.as_array((s_t * cols).from_address(src + r * src_strides[0] * ctypes.sizeof(s_t)))
            out = np.ctypeslib.as_array((d_t * cols).from_address(dst + r * dst_strides[0] * ctypes.sizeof(d_t)))
            if (sk, dk) == ("f32", "bf16"):
                out[:] = R.f32_to_bf16_bits(row)
            elif (sk, dk) == ("bf16", "f32"):
                out[:] = R.bf16_bits_to_f32(row)
            else:
                raise AssertionError((sk, dk))


def test_direct_casts_plan_the_boxes_torch_copies():
    """A fused qkv parameter in bf16 fed from fp32 q / k / v sources that are each published as
    row shards, and an fp32 parameter fed from a bf16 source through a column window: the boxes
    `plan_transfer_2d(fuse_casts=True)` returns, executed on the host, equal the engine's own
    `copy_` (the reference casts the same copies after staging, transfer_plan.py:49-60)."""
    from modelexpress_b200.geometry import capture_geometry
    from modelexpress_b200.planner import DirectCast, ShardSpec, SourceSpec, plan_transfer_2d

    h, q, kv, tp, rank = 64, 96, 32, 2, 1

    class Engine(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.qkv = torch.nn.Parameter(torch.zeros((q + 2 * kv) // tp, h, dtype=torch.bfloat16))
            self.wide = torch.nn.Parameter(torch.zeros(40, h // tp, dtype=torch.float32))

        def load_weights(self, weights):
            for name, w in weights:
                if name in ("q", "k", "v"):
                    n = (q if name == "q" else kv) // tp
                    at = {"q": 0, "k": q // tp, "v": (q + kv) // tp}[name]
                    self.qkv.data[at: at + n].copy_(w[rank * n: (rank + 1) * n])
                elif name == "wide":
                    self.wide.data.copy_(w[:, rank * (h // tp): (rank + 1) * (h // tp)])

    rng = np.random.default_rng(8)
    full = {"q": rng.standard_normal((q, h)).astype(np.float32), "k": rng.standard_normal((kv, h)).astype(np.float32),
            "v": rng.standard_normal((kv, h)).astype(np.float32)}
    wide_bits = rng.integers(0, 0x7F00, size=(40, h), dtype=np.uint16)
    truth = Engine()
    truth.load_weights([(n, torch.from_numpy(a)) for n, a in full.items()]
                       + [("wide", torch.from_numpy(wide_bits.view(np.int16)).view(torch.bfloat16))])
    sources = {}
    for n, a in full.items():        # four row shards each
        per = a.shape[0] // 4
        sources[n] = SourceSpec(a.shape, torch.float32, 4,
                                [ShardSpec((s * per, 0), (per, h), "t", a[s * per:].ctypes.data, 4) for s in range(4)])
    sources["wide"] = SourceSpec((40, h), torch.bfloat16, 2, [ShardSpec((0, 0), (40, h), "t", wide_bits.ctypes.data, 2)])
    model = Engine()
    manifest = [(n, s.dtype, tuple(s.global_shape)) for n, s in sources.items()]
    cap = capture_geometry(model, manifest, model.load_weights, device=torch.device("cpu"))
    assert not cap.unsupported_reasons
    dests = {n: p.data for n, p in model.named_parameters()}
    table, not_planned, converts = plan_transfer_2d(cap.copies, sources, lambda n: dests[n].data_ptr(), None,
                                                    fuse_casts=True, dst_elsize=lambda n: dests[n].element_size())
    assert len(table) == 0 and not not_planned
    assert all(isinstance(c, DirectCast) for c in converts) and len(converts) == 4
    assert sum(c.nbytes for c in converts) == sum(a.nbytes for a in full.values()) // tp + 40 * (h // tp) * 2
    for c in converts:
        _run_boxes_on_host(c.boxes)
    for n, p in truth.named_parameters():
        assert torch.equal(dests[n].view(torch.int16 if p.dtype == torch.bfloat16 else torch.int32),
                           p.data.view(torch.int16 if p.dtype == torch.bfloat16 else torch.int32)), n
