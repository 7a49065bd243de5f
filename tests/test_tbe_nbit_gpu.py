"""GPU parity: quantised-inference TBE forward through the C ABI vs the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle
from tests import helpers
from torchlib_xpu_b200 import cabi, workloads

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-3, 1e-3   # int8 / int4 pooling, fp16 output


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _run(W, wo, tys, Do, rows, B, indices, offsets, psw, pooling, out_dtype, row_alignment,
         tell_types=True):
    """tell_types: pass the set of table types along (the call may then skip the kernel of the types
    that are absent); the result must not depend on it."""
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = cabi.nbit_forward(_dev(W), _dev(wo), _dev(tys), _dev(Do), int(Do[-1]),
                            int(np.max(np.diff(Do))), _dev(indices), _dev(offsets), B, pooling,
                            None if psw is None else _dev(psw), out_dtype, row_alignment,
                            _dev(np.asarray(rows, dtype=np.int64)), status,
                            table_types=set(int(t) for t in tys) if tell_types else None)
    torch.cuda.synchronize()
    return out, int(status.item())


@pytest.mark.parametrize("row_alignment", [16, 1])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("pooling", [oracle.SUM, oracle.MEAN])
@pytest.mark.parametrize("weighted", [False, True])
def test_nbit_mixed_tables(row_alignment, out_dtype, pooling, weighted):
    rng = workloads.rng_for(300)
    tys = [oracle.INT8, oracle.INT4, oracle.INT8, oracle.INT4, oracle.INT2, oracle.FP16,
           oracle.FP32, oracle.INT8, oracle.INT4, oracle.INT4]
    Ds = [128, 128, 64, 256, 64, 128, 32, 20, 36, 1024]
    rows = [90, 80, 70, 60, 50, 40, 30, 20, 25, 12]
    T, B = len(tys), 41
    W, wo, Do, tys_a = helpers.quantised_tables(rng, rows, Ds, tys, row_alignment)
    _, offsets, indices = helpers.ragged_bags(rng, T, B, rows, 0, 50, empty_fraction=0.1)
    psw = rng.random(indices.size).astype(np.float32) if weighted else None
    want = oracle.nbit_forward(W, wo, tys_a, Do, row_alignment, B, indices, offsets, psw, pooling)
    got, status = _run(W, wo, tys_a, Do, rows, B, indices, offsets, psw, pooling, out_dtype,
                       row_alignment)
    assert status == 0
    np.testing.assert_allclose(got.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL)


def test_nbit_single_row_bags_are_plain_dequantisation():
    """One row per bag, fp32 out: q*scale + bias per element, to fp32 rounding."""
    rng = workloads.rng_for(301)
    for ty, D in ((oracle.INT8, 128), (oracle.INT4, 128), (oracle.INT4, 64), (oracle.INT8, 256)):
        rows = 64
        W, wo, Do, tys_a = helpers.quantised_tables(rng, [rows], [D], [ty], 16)
        indices, offsets = rng.permutation(rows).astype(np.int64), np.arange(rows + 1, dtype=np.int64)
        want = oracle.nbit_forward(W, wo, tys_a, Do, 16, rows, indices, offsets)
        got, status = _run(W, wo, tys_a, Do, [rows], rows, indices, offsets, None, oracle.SUM,
                           torch.float32, 16)
        assert status == 0
        np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-6, atol=1e-6)


def test_nbit_flags_out_of_range_indices():
    rng = workloads.rng_for(302)
    W, wo, Do, tys_a = helpers.quantised_tables(rng, [30], [128], [oracle.INT4], 16)
    _, offsets, indices = helpers.ragged_bags(rng, 1, 6, [30], 2, 5)
    bad = indices.copy()
    bad[1] = 30
    got, status = _run(W, wo, tys_a, Do, [30], 6, bad, offsets, None, oracle.SUM, torch.float32, 16)
    assert status & cabi.DEV_INDEX_OUT_OF_RANGE
    keep = np.ones(indices.size, dtype=np.float32)
    keep[1] = 0
    want = oracle.nbit_forward(W, wo, tys_a, Do, 16, 6, np.where(keep > 0, indices, 0), offsets, keep)
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-5, atol=1e-5)


def test_nbit_named_config_scaled_down_against_oracle():
    """The quantised configuration's shape (half INT8, half INT4, D=128, L~U{1..100}, Zipf 1.1,
    fp16 out) with fewer tables and rows, against the oracle."""
    T, E, D, B = 8, 50_000, 128, 1024
    inp = workloads.tbe_inputs(T, B, E, D, 1, 100, 3, "zipf", 1.1)
    rng = workloads.rng_for(3000)
    tys = [oracle.INT8 if t < T // 2 else oracle.INT4 for t in range(T)]
    W, wo, Do, tys_a = helpers.quantised_tables(rng, [E] * T, [D] * T, tys, 16)
    want = oracle.nbit_forward(W, wo, tys_a, Do, 16, B, inp.indices, inp.offsets)
    got, status = _run(W, wo, tys_a, Do, [E] * T, B, inp.indices, inp.offsets, None, oracle.SUM,
                       torch.float16, 16)
    assert status == 0
    np.testing.assert_allclose(got.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    blind, status = _run(W, wo, tys_a, Do, [E] * T, B, inp.indices, inp.offsets, None, oracle.SUM,
                         torch.float16, 16, tell_types=False)
    assert status == 0 and torch.equal(blind, got)


@pytest.mark.parametrize("ty,D", [(oracle.INT8, 128), (oracle.INT8, 4), (oracle.INT8, 68), (oracle.INT4, 128),
                                  (oracle.INT4, 8), (oracle.INT4, 72)])
@pytest.mark.parametrize("weighted", [False, True])
def test_nbit_register_gather_shapes(ty, D, weighted):
    """INT8 / INT4 rows of 4 ... 128 elements (the register-gather kernel, one or two code words per
    lane, some lanes idle), bags of 0 ... 70 rows with ids out of range mixed in, MEAN pooling."""
    rng = workloads.rng_for(310 + D)
    rows, B = [500, 37], 97
    W, wo, Do, tys_a = helpers.quantised_tables(rng, rows, [D, D], [ty, ty], 16)
    _, offsets, indices = helpers.ragged_bags(rng, 2, B, rows, 0, 70, empty_fraction=0.1)
    psw = rng.random(indices.size).astype(np.float32) if weighted else None
    want = oracle.nbit_forward(W, wo, tys_a, Do, 16, B, indices, offsets, psw, oracle.MEAN)
    got, status = _run(W, wo, tys_a, Do, rows, B, indices, offsets, psw, oracle.MEAN, torch.float32, 16)
    assert status == 0
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("weighted,pooling,idx_dtype,B", [
    (False, oracle.SUM, np.int64, 16001),      # groups of 3 bags, the last group short
    (True, oracle.MEAN, np.int32, 40000),      # groups of 8 (the most a warp takes)
    (False, oracle.MEAN, np.int32, 25013),
])
def test_nbit_groups_of_bags(weighted, pooling, idx_dtype, B):
    """A grid of more than about 47 k bags gives every warp a GROUP of consecutive bags to pool as one
    stream of lookups. INT8 and INT4 rows of 128, 64 and 20 / 40 elements (and a table of a type the
    register kernel leaves to the ring engine), bags of 0 to 40 lookups, runs of empty bags -- the tail
    of a table and whole groups included -- and ids out of range."""
    rng = workloads.rng_for(320 + B)
    tys = [oracle.INT8, oracle.INT4, oracle.INT8, oracle.INT4, oracle.INT2, oracle.INT8]
    Ds = [128, 128, 64, 40, 64, 20]
    rows = [3000, 2000, 1000, 500, 300, 600]
    T = len(Ds)
    W, wo, Do, tys_a = helpers.quantised_tables(rng, rows, Ds, tys, 16)
    lengths, _, _ = helpers.ragged_bags(rng, T, B, rows, 0, 40, empty_fraction=0.33)
    lengths[B - 40:B] = 0
    lengths[2 * B:2 * B + 64] = 0
    lengths[-5:] = 0
    offsets = np.zeros(T * B + 1, dtype=np.int64)
    np.cumsum(lengths, out=offsets[1:])
    indices = np.zeros(int(offsets[-1]), dtype=np.int64)
    for t in range(T):
        a, b = int(offsets[t * B]), int(offsets[(t + 1) * B])
        indices[a:b] = rng.integers(0, rows[t], size=b - a, dtype=np.int64)
    bad_at = rng.choice(indices.size, size=200, replace=False)
    bad = indices.copy()
    bad[bad_at[:100]] = 5000               # past every table
    bad[bad_at[100:]] = -1
    psw = rng.random(indices.size).astype(np.float32) if weighted else None
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = cabi.nbit_forward(_dev(W), _dev(wo), _dev(tys_a), _dev(Do), int(Do[-1]), int(np.max(np.diff(Do))),
                            _dev(bad.astype(idx_dtype)), _dev(offsets.astype(idx_dtype)), B, pooling,
                            None if psw is None else _dev(psw), torch.float32, 16,
                            _dev(np.asarray(rows, dtype=np.int64)), status)
    torch.cuda.synchronize()
    assert int(status.item()) & cabi.DEV_INDEX_OUT_OF_RANGE
    # flagged lookups contribute nothing (MEAN still divides by the bag's length)
    keep = np.ones(indices.size, dtype=np.float32)
    keep[bad_at] = 0.0
    want = oracle.nbit_forward(W, wo, tys_a, Do, 16, B, np.where(keep > 0, indices, 0), offsets,
                               keep if psw is None else psw * keep, pooling)
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=RTOL, atol=ATOL)
