"""The box-convert kernel against torch's strided device copy: the step the reference leaves
to ``dst.copy_(staged)`` after a pull (refit/reshard/receiver.py:964-971) and its permuted
boxes (refit/reshard/slice_plan.py:170-224).  Bit-exact, NaN payloads included."""

import itertools

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

KIND = {"float32": "f32", "float16": "f16", "bfloat16": "bf16"}
BITS = {1: "uint8", 2: "int16", 4: "int32", 8: "int64"}


def _ctx():
    from modelexpress_b200.runtime import Context

    return Context([0])


def _random_values(torch, n, dtype, seed):
    """Every bit pattern class of the dtype: random bits (NaNs, infinities, subnormals included)."""
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    size = torch.empty((), dtype=dtype).element_size()
    raw = torch.randint(0, 256, (n * size,), dtype=torch.uint8, device="cuda", generator=g)
    return raw.view(dtype)


def _bits(torch, t):
    return t.contiguous().view(getattr(torch, BITS[t.element_size()]))


def _run(torch, ctx, src, dst, extents, strides, offset=0):
    """Kernel into ``dst``; torch's own strided copy into a clone; compare every byte of both."""
    want = dst.clone()
    torch.as_strided(want, extents, strides, offset).copy_(src.reshape(extents))
    torch.cuda.synchronize()
    same = src.dtype == dst.dtype
    sk = "raw" if same else KIND[str(src.dtype).split(".")[1]]
    dk = "raw" if same else KIND[str(dst.dtype).split(".")[1]]
    moved = ctx.convert_boxes([(src.data_ptr(), dst.data_ptr() + offset * dst.element_size(), extents, strides,
                                sk, dk, src.element_size())], 0)
    n = int(np.prod(extents)) if len(extents) else 1
    assert moved == n * (src.element_size() + dst.element_size())
    assert torch.equal(_bits(torch, dst), _bits(torch, want))


@pytest.mark.parametrize("pair", [("float32", "bfloat16"), ("float32", "float16"), ("bfloat16", "float32"),
                                  ("float16", "float32"), ("bfloat16", "float16"), ("float16", "bfloat16")])
def test_casts_match_torch_bit_for_bit(pair):
    import torch

    ctx = _ctx()
    sd, dd = getattr(torch, pair[0]), getattr(torch, pair[1])
    for n, shift in ((1 << 20, 0), (100003, 0), (4099, 3), (7, 1), (1, 0)):
        src_all = _random_values(torch, n + 8, sd, 11 + n)
        # the special values by name as well
        special = torch.tensor([0.0, -0.0, float("inf"), float("-inf"), float("nan"), 65504.0, 65520.0,
                                1e-8, -1e-40, 3.3895313892515355e38], dtype=torch.float32, device="cuda")
        k = min(n, special.numel())
        src_all[shift: shift + k] = special[:k].to(sd) if sd != torch.float32 else special[:k]
        src = src_all[shift: shift + n]
        dst_all = torch.zeros(n + 8, dtype=dd, device="cuda")
        _run(torch, ctx, src, dst_all, [n], [1], offset=shift)
    ctx.close()


@pytest.mark.parametrize("size", [1, 2, 4, 8])
def test_transposes_of_every_element_size(size):
    import torch

    ctx = _ctx()
    dtype = getattr(torch, BITS[size])
    for m, n in ((64, 64), (1000, 3000), (129, 67), (2, 4096), (4096, 2), (770, 1538)):
        src = _random_values(torch, m * n, dtype, m * 7 + n)
        dst = torch.zeros(n * m, dtype=dtype, device="cuda")
        _run(torch, ctx, src, dst, [m, n], [1, m])          # dst is [n, m] contiguous
        # into a column window of a wider parameter [n, m + 10], two columns in
        wide = torch.zeros(n * (m + 10), dtype=dtype, device="cuda")
        _run(torch, ctx, src, wide, [m, n], [1, m + 10], offset=2)
        _run(torch, ctx, src, wide, [m, n], [1, m + 10], offset=3)   # odd offset: no element pairs
    ctx.close()


def test_transposed_casts_and_higher_ranks():
    import torch

    ctx = _ctx()
    # a stack of experts stored [E, I, H] landing as [E, H, I] in fp32 (transposed and widened)
    e, i, h = 6, 320, 192
    src = _random_values(torch, e * i * h, torch.bfloat16, 3)
    dst = torch.zeros(e * h * i, dtype=torch.float32, device="cuda")
    _run(torch, ctx, src, dst, [e, i, h], [h * i, 1, i])
    # narrowed on the way
    src = _random_values(torch, e * i * h, torch.float32, 4)
    dst = torch.zeros(e * h * i, dtype=torch.bfloat16, device="cuda")
    _run(torch, ctx, src, dst, [e, i, h], [h * i, 1, i])
    # every permutation of a rank-4 box, raw two-byte elements; extents chosen odd and even
    shape = (3, 10, 34, 66)
    src = _random_values(torch, int(np.prod(shape)), torch.int16, 5)
    for perm in itertools.permutations(range(4)):
        out_shape = [shape[p] for p in perm]
        out_strides = [int(np.prod(out_shape[k + 1:])) for k in range(4)]
        strides = [0] * 4
        for k, p in enumerate(perm):
            strides[p] = out_strides[k]
        dst = torch.zeros(int(np.prod(shape)), dtype=torch.int16, device="cuda")
        _run(torch, ctx, src, dst, list(shape), strides)
    # no unit-stride dim at all in the destination (every second element), with a cast
    src = _random_values(torch, 33 * 65, torch.float16, 6)
    dst = torch.zeros(33 * 65 * 2, dtype=torch.float32, device="cuda")
    _run(torch, ctx, src, dst, [33, 65], [130, 2])
    # rank 0 and empty boxes
    one = _random_values(torch, 1, torch.float32, 7)
    out = torch.zeros(1, dtype=torch.bfloat16, device="cuda")
    _run(torch, ctx, one, out, [], [])
    assert ctx.convert_boxes([(one.data_ptr(), out.data_ptr(), [0, 4], [4, 1], "f32", "bf16", 4)], 0) == 0
    ctx.close()


def test_strided_sources_are_read_in_place():
    """A box whose source is a strided slice of a larger tensor (a shard read where it lies):
    a column window of a wider fp32 matrix cast into a bf16 parameter, the same window
    transposed, and a window whose rows start off every vector boundary."""
    import torch

    ctx = _ctx()
    rows, width = 700, 1000
    full = _random_values(torch, rows * width, torch.float32, 21).reshape(rows, width)
    for c0, cols in ((0, 1000), (8, 512), (3, 333), (996, 4)):
        win = full[:, c0: c0 + cols]
        src_ptr = full.data_ptr() + c0 * 4
        # plain cast into a window of a wider bf16 parameter
        dst = torch.zeros(rows, width + 24, dtype=torch.bfloat16, device="cuda")
        want = dst.clone()
        want[:, 16: 16 + cols].copy_(win)
        ctx.convert_boxes([(src_ptr, dst.data_ptr() + 16 * 2, [rows, cols], [width + 24, 1], "f32", "bf16", 4,
                            [width, 1])], 0)
        assert torch.equal(_bits(torch, dst), _bits(torch, want)), (c0, cols)
        # transposed on the way
        dst_t = torch.zeros(cols, rows, dtype=torch.bfloat16, device="cuda")
        ctx.convert_boxes([(src_ptr, dst_t.data_ptr(), [rows, cols], [1, rows], "f32", "bf16", 4, [width, 1])], 0)
        assert torch.equal(_bits(torch, dst_t), _bits(torch, win.t().to(torch.bfloat16)))
        # moved unchanged
        raw = torch.zeros(rows, cols, dtype=torch.float32, device="cuda")
        ctx.convert_boxes([(src_ptr, raw.data_ptr(), [rows, cols], [cols, 1], "raw", "raw", 4, [width, 1])], 0)
        assert torch.equal(_bits(torch, raw), _bits(torch, win))
    # a source whose inner dim is not unit-stride is refused
    from modelexpress_b200._lib import MxbError

    with pytest.raises(MxbError) as e:
        ctx.convert_boxes([(full.data_ptr(), full.data_ptr(), [10, 10], [10, 1], "raw", "raw", 4, [1, width])], 0)
    assert e.value.code == -9
    ctx.close()


def test_kernel_matches_the_oracle():
    """Through the C ABI against the CPU restatement (oracle.ref_port.box_convert): a permuted
    rank-3 box of two-byte elements and a transposed fp32 -> bf16 window of a wider parameter."""
    import torch

    from oracle import ref_port as R

    ctx = _ctx()
    rng = np.random.default_rng(12)
    shape = (5, 70, 130)
    src = rng.integers(0, 1 << 15, size=int(np.prod(shape)), dtype=np.int16)
    strides = [70, 1, 5 * 70]                       # destination laid out [130, 5, 70]
    want = np.zeros(src.size, dtype=np.int16)
    R.box_convert(src, shape, strides, want)
    d_src = torch.from_numpy(src).cuda()
    d_dst = torch.zeros(src.size, dtype=torch.int16, device="cuda")
    torch.cuda.synchronize()
    ctx.convert_boxes([(d_src.data_ptr(), d_dst.data_ptr(), list(shape), strides, "raw", "raw", 2)], 0)
    assert np.array_equal(d_dst.cpu().numpy(), want)
    m, n = 300, 516
    x = rng.standard_normal(m * n).astype(np.float32)
    want = np.zeros(n * (m + 4), dtype=np.uint16)
    R.box_convert(x, (m, n), (1, m + 4), want, dst_offset=4, cast=R.f32_to_bf16_bits)
    d_x = torch.from_numpy(x).cuda()
    d_out = torch.zeros(n * (m + 4), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    ctx.convert_boxes([(d_x.data_ptr(), d_out.data_ptr() + 8, [m, n], [1, m + 4], "f32", "bf16", 4)], 0)
    assert np.array_equal(d_out.view(torch.int16).cpu().numpy().view(np.uint16), want)
    ctx.close()


def test_many_boxes_one_call_and_rejections():
    import torch

    from modelexpress_b200._lib import MxbError

    ctx = _ctx()
    boxes, checks, alive = [], [], []
    for k in range(40):
        m, n = 16 + 13 * k, 24 + 5 * k
        src = _random_values(torch, m * n, torch.float32, 100 + k)
        alive.append(src)
        if k % 2:
            dst = torch.zeros(m * n, dtype=torch.bfloat16, device="cuda")
            boxes.append((src.data_ptr(), dst.data_ptr(), [m, n], [1, m], "f32", "bf16", 4))
            checks.append((dst, src.reshape(m, n).t().contiguous().to(torch.bfloat16).reshape(-1)))
        else:
            dst = torch.zeros(m * n, dtype=torch.float32, device="cuda")
            boxes.append((src.data_ptr(), dst.data_ptr(), [m * n], [1], "raw", "raw", 4))
            checks.append((dst, src))
    torch.cuda.synchronize()
    before = ctx.launch_count
    ctx.convert_boxes(boxes, 0)
    assert ctx.launch_count == before + 2      # one launch per conversion present: moves and fp32 -> bf16
    for got, want in checks:
        assert torch.equal(_bits(torch, got), _bits(torch, want))
    src = torch.zeros(64, dtype=torch.float32, device="cuda")
    with pytest.raises(MxbError) as e:     # a pair of kinds outside the table
        ctx.convert_boxes([(src.data_ptr(), src.data_ptr(), [4], [1], "raw", "f32", 4)], 0)
    assert e.value.code == -9
    with pytest.raises(MxbError) as e:     # five dims that do not merge
        ctx.convert_boxes([(src.data_ptr(), src.data_ptr(), [2, 2, 2, 2, 2], [1, 2, 4, 8, 16], "raw", "raw", 1)], 0)
    assert e.value.code == -9
    with pytest.raises(MxbError):          # an address off its element's alignment
        ctx.convert_boxes([(src.data_ptr() + 2, src.data_ptr(), [4], [1], "f32", "bf16", 4)], 0)
    ctx.close()


def test_apply_converts_takes_the_kernel_on_the_gpu():
    """planner.apply_converts: a staged transposed box and a plain cast go through one call."""
    import torch

    from modelexpress_b200.planner import ConvertSpec, apply_converts

    ctx = _ctx()
    i, h = 96, 160
    box = _random_values(torch, i * h, torch.bfloat16, 9)            # source [I, H]
    gate = _random_values(torch, 64 * 32, torch.bfloat16, 10)         # source [64, 32], served bf16
    staging = torch.zeros(box.numel() * 2 + 256 + gate.numel() * 2, dtype=torch.uint8, device="cuda")
    off2 = (box.numel() * 2 + 255) // 256 * 256
    staging[: box.numel() * 2] = box.view(torch.uint8)
    staging[off2: off2 + gate.numel() * 2] = gate.view(torch.uint8)
    w = torch.zeros(h, i, dtype=torch.bfloat16, device="cuda")          # parameter stored [H, I]
    r = torch.zeros(64, 32, dtype=torch.float32, device="cuda")         # parameter kept in fp32
    converts = [ConvertSpec("w", (h, i), (i, 1), 0, torch.bfloat16, 0, box.numel() * 2, (i, h), (1, 0)),
                ConvertSpec("r", (64, 32), (32, 1), 0, torch.bfloat16, off2, gate.numel() * 2)]
    torch.cuda.synchronize()
    before = ctx.launch_count
    apply_converts(converts, staging, {"w": w, "r": r}, ctx)
    assert ctx.launch_count == before + 2      # the two-byte move and the bf16 -> fp32 cast
    assert torch.equal(_bits(torch, w), _bits(torch, box.reshape(i, h).t().contiguous()))
    assert torch.equal(_bits(torch, r), _bits(torch, gate.reshape(64, 32).float()))
    ctx.close()
