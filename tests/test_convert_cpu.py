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
