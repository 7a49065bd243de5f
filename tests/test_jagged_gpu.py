"""GPU parity: jagged kernels through the C ABI vs the CPU oracle. Bit-exact."""
import numpy as np
import pytest
import torch

import oracle
from torchlib_xpu_b200 import cabi, workloads

pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _bits(t):
    return t.cpu().contiguous().view(torch.uint8).numpy()


CASES = [
    # B, max_L, D, dtype, offset dtype, length cap (above max_L => truncation)
    (64, 16, 32, np.float32, np.int64, 16),
    (33, 7, 5, np.float32, np.int64, 11),      # odd D: 4-byte vectors, truncated rows
    (40, 9, 6, np.float16, np.int32, 9),       # 12-byte rows: 4-byte vectors
    (17, 5, 3, np.float16, np.int64, 8),       # 6-byte rows: 2-byte vectors
    (25, 6, 7, np.uint8, np.int64, 6),         # 1-byte vectors
    (19, 4, 3, np.int64, np.int32, 6),         # 8-byte elements
    (1, 1, 1, np.float32, np.int64, 1),
    (512, 128, 256, np.float32, np.int64, 128),  # the named config's row shape
]


@pytest.mark.parametrize("B,max_L,D,dtype,odtype,cap", CASES)
def test_jagged_roundtrip_and_add(B, max_L, D, dtype, odtype, cap):
    rng = workloads.rng_for(100 + B)
    lengths = rng.integers(0, cap + 1, size=B, dtype=np.int64)
    offsets = np.zeros(B + 1, dtype=np.int64)
    np.cumsum(lengths, out=offsets[1:])
    total = int(offsets[-1])
    if np.issubdtype(dtype, np.floating):
        values = rng.standard_normal((total, D)).astype(dtype)
        pad = -2.5
    else:
        values = rng.integers(0, 120, size=(total, D)).astype(dtype)
        pad = 7
    d_off = _dev(offsets.astype(odtype))
    d_values = _dev(values)

    dense = cabi.jagged_to_padded_dense(d_values, [d_off], [max_L], pad)
    want = oracle.jagged_to_padded_dense(values, [offsets], [max_L], pad)
    assert np.array_equal(_bits(dense), want.view(np.uint8).reshape(-1)) or \
        np.array_equal(_bits(dense).reshape(-1), want.view(np.uint8).reshape(-1))

    back = cabi.dense_to_jagged(dense, [d_off], total)
    want_back = oracle.dense_to_jagged(want, [offsets], total)
    assert np.array_equal(_bits(back).reshape(-1), want_back.view(np.uint8).reshape(-1))

    if dtype in (np.float32, np.float16):
        y = rng.standard_normal((B, max_L, D)).astype(dtype)
        out = cabi.jagged_dense_elementwise_add(d_values, [d_off], _dev(y))
        if dtype == np.float32:
            want_add = oracle.jagged_dense_elementwise_add(values, [offsets], y)
        else:
            want_add = (oracle.jagged_to_padded_dense(values, [offsets], [max_L], 0).astype(np.float32)
                        + y.astype(np.float32)).astype(np.float16)
        assert np.array_equal(_bits(out).reshape(-1), want_add.view(np.uint8).reshape(-1))


def test_jagged_bf16_add():
    rng = workloads.rng_for(131)
    j = workloads.jagged_inputs(48, 12, 24, 131)
    x = torch.from_numpy(rng.standard_normal((j.total_rows, j.D)).astype(np.float32)).bfloat16()
    y = torch.from_numpy(rng.standard_normal((j.B, j.max_L, j.D)).astype(np.float32)).bfloat16()
    off = torch.from_numpy(j.offsets)
    out = cabi.jagged_dense_elementwise_add(x.cuda(), [off.cuda()], y.cuda())
    want = (torch.ops.aten._jagged_to_padded_dense_forward(x.float(), [off], [j.max_L], 0.0)
            + y.float()).bfloat16()
    assert torch.equal(out.cpu().view(torch.int16), want.view(torch.int16))


def test_jagged_nested_offsets():
    rng = workloads.rng_for(132)
    outer = 37
    l1 = rng.integers(0, 6, size=outer)
    o1 = np.zeros(outer + 1, dtype=np.int64)
    np.cumsum(l1, out=o1[1:])
    l2 = rng.integers(0, 9, size=o1[-1])
    o2 = np.zeros(o1[-1] + 1, dtype=np.int64)
    np.cumsum(l2, out=o2[1:])
    values = rng.standard_normal((o2[-1], 12)).astype(np.float32)
    max_lengths = [4, 6]
    d_offs = [_dev(o1), _dev(o2)]
    dense = cabi.jagged_to_padded_dense(_dev(values), d_offs, max_lengths, 9.0)
    want = oracle.jagged_to_padded_dense(values, [o1, o2], max_lengths, 9.0)
    assert np.array_equal(dense.cpu().numpy(), want)
    back = cabi.dense_to_jagged(dense, d_offs, int(o2[-1]))
    assert np.array_equal(back.cpu().numpy(), oracle.dense_to_jagged(want, [o1, o2], int(o2[-1])))
    y = rng.standard_normal(want.shape).astype(np.float32)
    out = cabi.jagged_dense_elementwise_add(_dev(values), d_offs, _dev(y))
    assert np.array_equal(out.cpu().numpy(), oracle.jagged_dense_elementwise_add(values, [o1, o2], y))


def test_jagged_empty_inputs():
    off = torch.zeros(5, dtype=torch.int64, device="cuda")
    values = torch.zeros((0, 8), dtype=torch.float32, device="cuda")
    dense = cabi.jagged_to_padded_dense(values, [off], [3], 1.5)
    assert dense.shape == (4, 3, 8) and torch.all(dense == 1.5)
    back = cabi.dense_to_jagged(dense, [off], 0)
    assert back.shape == (0, 8)
    none = cabi.jagged_to_padded_dense(values, [torch.zeros(1, dtype=torch.int64, device="cuda")], [3], 0.0)
    assert none.shape == (0, 3, 8)


def test_jagged_full_config_properties():
    """The named jagged configuration at full size: size-independent properties."""
    cfg = workloads.CONFIGS["jagged"]
    j = workloads.jagged_inputs(cfg["B"], cfg["max_L"], cfg["D"], cfg["seed"])
    gen = torch.Generator(device="cuda").manual_seed(1)
    values = torch.randn((j.total_rows, j.D), device="cuda", generator=gen)
    y = torch.randn((j.B, j.max_L, j.D), device="cuda", generator=gen)
    off = torch.from_numpy(j.offsets).cuda()
    dense = cabi.jagged_to_padded_dense(values, [off], [j.max_L], 0.0)
    # round trip is the identity on values; padding positions are exactly the pad value
    assert torch.equal(cabi.dense_to_jagged(dense, [off], j.total_rows), values)
    lengths = torch.from_numpy(j.lengths).cuda()
    mask = torch.arange(j.max_L, device="cuda")[None, :] < lengths[:, None]
    assert torch.all(dense[~mask] == 0)
    assert torch.equal(dense.sum(dtype=torch.float64), values.sum(dtype=torch.float64)) or \
        torch.allclose(dense.sum(dtype=torch.float64), values.sum(dtype=torch.float64))
    # add == to_dense + y, bit for bit
    assert torch.equal(cabi.jagged_dense_elementwise_add(values, [off], y), dense + y)
    # a sampled slice against the oracle
    rows = slice(0, 64)
    want = oracle.jagged_to_padded_dense(values[:int(j.offsets[64])].cpu().numpy(),
                                         [j.offsets[:65]], [j.max_L], 0.0)
    assert np.array_equal(dense[rows].cpu().numpy(), want)
