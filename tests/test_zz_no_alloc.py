"""The allocation-free sort entry point (b200tbe_radix_sort_pairs_static) against the ordinary one.

Some users of the library cannot allocate device memory at call time -- a C host without a tensor
allocator, a server whose HBM is already fully committed to tables, a loop that must avoid the
device synchronisation of cudaMalloc -- so this entry point keeps its scratch in a fixed array inside
the library. The file name makes pytest collect it last: a run that stops at the first failure has
then already run every other test."""
import ctypes

import numpy as np
import pytest
import torch

from torchlib_xpu_b200 import cabi, workloads

pytestmark = pytest.mark.gpu


def _sort_static(keys, vals, bits, outs=None):
    """Calls the entry point through the C ABI with raw pointers; the outputs are ordinary tensors
    the caller owns (the entry point itself allocates nothing)."""
    keys_out, vals_out = outs if outs is not None else (torch.empty_like(keys), torch.empty_like(vals))
    st = cabi.lib().b200tbe_radix_sort_pairs_static(
        keys.data_ptr(), vals.data_ptr(), keys_out.data_ptr(), vals_out.data_ptr(), keys.numel(),
        keys.element_size(), bits, torch.cuda.current_stream().cuda_stream)
    return st, keys_out, vals_out


def test_static_sort_matches_the_ordinary_entry_point_twice_in_a_row():
    rng = workloads.rng_for(900)
    limit = int(cabi.lib().b200tbe_radix_sort_pairs_static_max())
    assert limit == 1 << 20
    # two calls in a row with different sizes and key widths share the scratch array
    for n, dtype, bits in ((300_001, np.int32, 25), (limit, np.int64, 37), (4097, np.int32, 9)):
        keys = rng.integers(0, 1 << min(bits, 62), size=n, dtype=np.int64)
        keys[rng.random(n) < 0.3] = keys[0]
        vals = np.arange(n, dtype=np.int32)
        k_dev = torch.from_numpy(keys.astype(dtype)).cuda()
        v_dev = torch.from_numpy(vals).cuda()
        want_k, want_v = cabi.radix_sort_pairs(k_dev.clone(), v_dev.clone(), bits)
        k_in, v_in = k_dev.clone(), v_dev.clone()
        outs = (torch.empty_like(k_in), torch.empty_like(v_in))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        st, got_k, got_v = _sort_static(k_in, v_in, bits, outs)
        torch.cuda.synchronize()
        # every buffer was in place before the call: the device's free memory must not have moved
        assert torch.cuda.mem_get_info()[0] >= free_before
        assert st == 0
        # integer work: bit-exact, as in the other sort tests: against the ordinary entry point ...
        assert torch.equal(got_k, want_k) and torch.equal(got_v, want_v)
        # ... and against a stable CPU sort of the same pairs
        order = np.argsort(keys.astype(np.uint64) & np.uint64((1 << bits) - 1), kind="stable")
        assert np.array_equal(got_k.cpu().numpy(), keys.astype(dtype)[order])
        assert np.array_equal(got_v.cpu().numpy(), vals[order])


def test_static_sort_rejects_sizes_beyond_its_capacity():
    limit = int(cabi.lib().b200tbe_radix_sort_pairs_static_max())
    n = limit + 1
    keys = torch.zeros(n, dtype=torch.int32, device="cuda")
    vals = torch.zeros(n, dtype=torch.int32, device="cuda")
    st, _, _ = _sort_static(keys, vals, 8)
    assert st == -5  # B200TBE_ERR_TOO_LARGE
    assert b"capacity" in cabi.lib().b200tbe_status_string(st)
    assert cabi.lib().b200tbe_radix_sort_pairs_static(None, None, None, None, -1, 4, 8, None) == -1
