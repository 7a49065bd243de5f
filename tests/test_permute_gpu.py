"""GPU parity: b200tbe_permute_segments vs the oracle's numpy segment permutation (byte work: exact)."""
import numpy as np
import pytest
import torch

import oracle
from torchlib_xpu_b200 import cabi, sharded, workloads

pytestmark = pytest.mark.gpu


def _want(values, lens, perm):
    """The oracle's permutation of the same inputs, on the host, as a CPU tensor."""
    return torch.from_numpy(oracle.permute_segments(values.cpu().numpy(), lens.cpu().numpy(), perm.cpu().numpy()))


def _case(rng, lengths, dtype):
    lengths = np.asarray(lengths, dtype=np.int64)
    total = int(lengths.sum())
    if np.issubdtype(dtype, np.floating):
        values = rng.standard_normal(total).astype(dtype)
    else:
        values = rng.integers(0, np.iinfo(dtype).max, size=total, dtype=dtype)
    perm = rng.permutation(lengths.size).astype(np.int64)
    return torch.from_numpy(values).cuda(), torch.from_numpy(lengths).cuda(), torch.from_numpy(perm).cuda()


@pytest.mark.parametrize("name", ["ragged", "tiny_segments", "whole_tables", "mostly_empty", "one_element"])
@pytest.mark.parametrize("dtype", [np.int64, np.int32, np.float32, np.float16])
def test_matches_reference(name, dtype):
    rng = workloads.rng_for(1200 + len(name))
    lengths = {
        "ragged": rng.integers(0, 60, size=5000),
        "tiny_segments": rng.integers(0, 2, size=40000),          # thousands of boundaries per tile
        "whole_tables": rng.integers(100000, 400000, size=7),     # segments far longer than a tile
        "mostly_empty": np.where(rng.random(30000) < 0.01, rng.integers(1, 3000, size=30000), 0),
        "one_element": [1],
    }[name]
    values, lens, perm = _case(rng, lengths, dtype)
    want = _want(values, lens, perm)
    got = sharded.kernel_permute_segments(values, lens, perm)
    assert torch.equal(got.cpu().view(torch.uint8), want.view(torch.uint8))


def test_int32_offsets_and_permutation_and_empty_input():
    rng = workloads.rng_for(1300)
    values, lens, perm = _case(rng, rng.integers(0, 40, size=3000), np.int64)
    want = _want(values, lens, perm)
    in_off = torch.zeros(lens.numel() + 1, dtype=torch.int32, device="cuda")
    in_off[1:] = torch.cumsum(lens, 0)
    out_off = torch.zeros_like(in_off)
    out_off[1:] = torch.cumsum(lens[perm], 0)
    got = cabi.permute_segments(values, in_off, out_off, perm.to(torch.int32))
    assert torch.equal(got.cpu(), want)
    empty = cabi.permute_segments(values[:0], in_off[:1], out_off[:1], perm[:0])
    assert empty.numel() == 0


def test_a_permutation_and_its_inverse_restore_the_input():
    rng = workloads.rng_for(1301)
    values, lens, perm = _case(rng, rng.integers(0, 300, size=20000), np.int64)
    once = sharded.kernel_permute_segments(values, lens, perm)
    inverse = torch.empty_like(perm)
    inverse[perm] = torch.arange(perm.numel(), device="cuda")
    back = sharded.kernel_permute_segments(once, lens[perm], inverse)
    assert torch.equal(back, values)
