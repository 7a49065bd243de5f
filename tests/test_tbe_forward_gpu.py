"""GPU parity: TBE forward (fp32 / fp16 tables) through the C ABI vs the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle
from tests import helpers
from torchlib_xpu_b200 import cabi, workloads

pytestmark = pytest.mark.gpu

RTOL_FP32 = 1e-5            # fp32 pooling
# Sums of up to ~70 terms of magnitude <= 1 that cancel to near zero differ between summation
# orders by a few ulps of the TERMS, not of the result: absolute slack of L * 2^-24.
ATOL_FP32_UNIT = 5e-6
RTOL_FP16, ATOL_FP16 = 1e-3, 1e-3   # fp16 tables or fp16 output


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _run(W, wo, Do, rows, B, indices, offsets, psw, pooling, out_dtype, idx_dtype=np.int64,
         check_bounds=True):
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = cabi.forward(
        _dev(W), _dev(wo), _dev(Do), int(Do[-1]), int(np.max(np.diff(Do))) if len(Do) > 1 else 0,
        _dev(indices.astype(idx_dtype)), _dev(offsets.astype(idx_dtype)), B, pooling,
        None if psw is None else _dev(psw), out_dtype,
        _dev(np.asarray(rows, dtype=np.int64)) if check_bounds else None, status)
    torch.cuda.synchronize()
    return out, int(status.item())


@pytest.mark.parametrize("wdtype", [np.float32, np.float16])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("pooling", [oracle.SUM, oracle.MEAN])
@pytest.mark.parametrize("weighted", [False, True])
def test_forward_mixed_dims(wdtype, out_dtype, pooling, weighted):
    rng = workloads.rng_for(200)
    # D = 128 (full warp or two rows per load), 64, 32, 8, 4, a non-vector 20 (fp16: 40 bytes), 256
    Ds = [128, 64, 32, 8, 4, 20, 256]
    rows = [300, 200, 100, 50, 40, 30, 60]
    T, B = len(Ds), 67
    W, wo, Do = helpers.float_tables(rng, rows, Ds, wdtype, -1.0, 1.0)
    _, offsets, indices = helpers.ragged_bags(rng, T, B, rows, 0, 45, empty_fraction=0.1)
    psw = rng.random(indices.size).astype(np.float32) if weighted else None
    ty = oracle.FP32 if wdtype == np.float32 else oracle.FP16
    want = oracle.tbe_forward(W, ty, wo, Do, B, indices, offsets, psw, pooling)
    got, status = _run(W, wo, Do, rows, B, indices, offsets, psw, pooling, out_dtype)
    assert status == 0
    if wdtype == np.float32 and out_dtype == torch.float32:
        np.testing.assert_allclose(got.cpu().numpy(), want, rtol=RTOL_FP32, atol=ATOL_FP32_UNIT)
    else:
        np.testing.assert_allclose(got.float().cpu().numpy(), want, rtol=RTOL_FP16, atol=ATOL_FP16)


@pytest.mark.parametrize("max_D", [512, 1024])
def test_forward_wide_rows(max_D):
    rng = workloads.rng_for(201)
    Ds, rows, B = [max_D, 128], [40, 40], 9
    W, wo, Do = helpers.float_tables(rng, rows, Ds, np.float32, -1, 1)
    _, offsets, indices = helpers.ragged_bags(rng, 2, B, rows, 0, 70)
    want = oracle.tbe_forward(W, oracle.FP32, wo, Do, B, indices, offsets)
    got, status = _run(W, wo, Do, rows, B, indices, offsets, None, oracle.SUM, torch.float32)
    assert status == 0
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=RTOL_FP32, atol=ATOL_FP32_UNIT)


def test_forward_int32_indices_and_long_bags():
    rng = workloads.rng_for(202)
    Ds, rows, B = [128, 128], [1000, 17], 5
    W, wo, Do = helpers.float_tables(rng, rows, Ds, np.float16, -1, 1)
    _, offsets, indices = helpers.ragged_bags(rng, 2, B, rows, 100, 700)
    want = oracle.tbe_forward(W, oracle.FP16, wo, Do, B, indices, offsets, None, oracle.MEAN)
    got, status = _run(W, wo, Do, rows, B, indices, offsets, None, oracle.MEAN, torch.float32,
                       idx_dtype=np.int32)
    assert status == 0
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=RTOL_FP16, atol=ATOL_FP16)


def test_forward_flags_out_of_range_indices():
    rng = workloads.rng_for(203)
    Ds, rows, B = [64], [50], 8
    W, wo, Do = helpers.float_tables(rng, rows, Ds, np.float32)
    _, offsets, indices = helpers.ragged_bags(rng, 1, B, rows, 1, 6)
    bad = indices.copy()
    bad[3] = 50       # one past the end
    bad[-1] = -4
    got, status = _run(W, wo, Do, rows, B, bad, offsets, None, oracle.SUM, torch.float32)
    assert status & cabi.DEV_INDEX_OUT_OF_RANGE
    # flagged lookups contribute nothing; everything else is as if they were absent
    keep = np.ones(indices.size, dtype=bool)
    keep[3] = keep[-1] = False
    psw = keep.astype(np.float32)
    safe = np.where(keep, indices, 0)
    want = oracle.tbe_forward(W, oracle.FP32, wo, Do, B, safe, offsets, psw)
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=RTOL_FP32, atol=1e-7)


@pytest.mark.parametrize("wdtype,weighted,pooling,idx_dtype,B", [
    (np.float16, False, oracle.SUM, np.int64, 12001),     # groups of 3 bags, the last group short
    (np.float16, True, oracle.MEAN, np.int32, 30000),     # groups of 7
    (np.float32, False, oracle.MEAN, np.int32, 30011),
    (np.float32, True, oracle.SUM, np.int64, 12001),
])
def test_forward_groups_of_bags(wdtype, weighted, pooling, idx_dtype, B):
    """A grid of more than about 47 k bags gives every warp a GROUP of consecutive bags to pool as one
    stream of lookups. Bags of 0 to 40 lookups, runs of empty bags (a third of all, the tail of a table
    included), rows of 16 to 512 bytes and one that is not a whole vector, ids out of range."""
    rng = workloads.rng_for(210 + B)
    Ds = [128, 64, 32, 8, 20, 4] if wdtype == np.float32 else [128, 64, 32, 8, 20, 256]
    rows = [3000, 2000, 1000, 500, 300, 600]
    T = len(Ds)
    W, wo, Do = helpers.float_tables(rng, rows, Ds, wdtype, -1.0, 1.0)
    lengths, _, _ = helpers.ragged_bags(rng, T, B, rows, 0, 40, empty_fraction=0.33)
    lengths[B - 40:B] = 0                  # a table that ends in empty bags
    lengths[2 * B:2 * B + 64] = 0          # whole groups without a lookup
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
    got, status = _run(W, wo, Do, rows, B, bad, offsets, psw, pooling, torch.float32, idx_dtype=idx_dtype)
    assert status & cabi.DEV_INDEX_OUT_OF_RANGE
    # flagged lookups contribute nothing (MEAN still divides by the bag's length)
    keep = np.ones(indices.size, dtype=np.float32)
    keep[bad_at] = 0.0
    ty = oracle.FP32 if wdtype == np.float32 else oracle.FP16
    want = oracle.tbe_forward(W, ty, wo, Do, B, np.where(keep > 0, indices, 0), offsets,
                              keep if psw is None else psw * keep, pooling)
    if wdtype == np.float32:
        np.testing.assert_allclose(got.cpu().numpy(), want, rtol=RTOL_FP32, atol=ATOL_FP32_UNIT)
    else:
        np.testing.assert_allclose(got.cpu().numpy(), want, rtol=RTOL_FP16, atol=ATOL_FP16)


def test_forward_empty_batch_and_bad_args():
    z = torch.zeros(1, dtype=torch.int64, device="cuda")
    out = cabi.forward(torch.zeros(4, device="cuda"), z, torch.zeros(2, dtype=torch.int32, device="cuda"),
                       0, 0, z, z, 0)
    assert out.shape == (0, 0)
    with pytest.raises(cabi.B200TbeError):
        cabi.forward(torch.zeros(4, device="cuda"), z, torch.zeros(2, dtype=torch.int32, device="cuda"),
                     4, 4, z.int(), z, 1)  # mixed index dtypes


def test_forward_scatter_to_destinations():
    """num_dests > 1: the batch is split across destination buffers at a column offset."""
    rng = workloads.rng_for(204)
    Ds, rows, B = [128, 64], [80, 80], 12
    W, wo, Do = helpers.float_tables(rng, rows, Ds, np.float16, -1, 1)
    _, offsets, indices = helpers.ragged_bags(rng, 2, B, rows, 0, 9)
    want = oracle.tbe_forward(W, oracle.FP16, wo, Do, B, indices, offsets)
    G, col0, stride = 3, 16, 16 + 192 + 8
    bufs = [torch.full((B // G, stride), -7.0, dtype=torch.float16, device="cuda") for _ in range(G)]
    cabi.forward(_dev(W), _dev(wo), _dev(Do), 192, 128, _dev(indices), _dev(offsets), B,
                 outputs=bufs, output_stride=stride, output_col_offset=col0, rows_per_dest=B // G,
                 output_dtype=torch.float16)
    torch.cuda.synchronize()
    for g, buf in enumerate(bufs):
        blk = buf.float().cpu().numpy()
        np.testing.assert_allclose(blk[:, col0:col0 + 192], want[g * (B // G):(g + 1) * (B // G)],
                                   rtol=RTOL_FP16, atol=ATOL_FP16)
        assert np.all(blk[:, :col0] == -7.0) and np.all(blk[:, col0 + 192:] == -7.0)


def test_forward_groups_of_bags_across_destinations():
    """Groups of bags with num_dests > 1: a destination's last row falls inside a group (rows_per_dest
    is not a multiple of the group size), so a warp moves on to the next buffer between two bags."""
    rng = workloads.rng_for(231)
    Ds, rows, B = [128, 64, 128, 32], [500, 400, 300, 200], 30011
    T = len(Ds)
    W, wo, Do = helpers.float_tables(rng, rows, Ds, np.float16, -1, 1)
    _, offsets, indices = helpers.ragged_bags(rng, T, B, rows, 0, 12, empty_fraction=0.2)
    want = oracle.tbe_forward(W, oracle.FP16, wo, Do, B, indices, offsets)
    G, rpd, total_D = 3, 10007, int(Do[-1])
    col0, stride = 8, 8 + total_D + 8
    bufs = [torch.full((rpd, stride), -7.0, dtype=torch.float16, device="cuda") for _ in range(G)]
    cabi.forward(_dev(W), _dev(wo), _dev(Do), total_D, max(Ds), _dev(indices), _dev(offsets), B,
                 outputs=bufs, output_stride=stride, output_col_offset=col0, rows_per_dest=rpd,
                 output_dtype=torch.float16)
    torch.cuda.synchronize()
    for g, buf in enumerate(bufs):
        blk = buf.float().cpu().numpy()
        n = min(rpd, B - g * rpd)
        np.testing.assert_allclose(blk[:n, col0:col0 + total_D], want[g * rpd:g * rpd + n], rtol=RTOL_FP16, atol=ATOL_FP16)
        assert np.all(blk[:, :col0] == -7.0) and np.all(blk[:, col0 + total_D:] == -7.0)
        assert np.all(blk[n:] == -7.0)


def test_forward_named_fp32_config_against_oracle():
    """T=8, E=100k, D=128 fp32, B=2048, L~U{1..40}, uniform ids, seed 0 -- full size."""
    cfg = workloads.CONFIGS["tbe_fp32_fwd"]
    inp = workloads.tbe_inputs(cfg["T"], cfg["B"], cfg["E"], cfg["D"], cfg["L_lo"], cfg["L_hi"],
                               cfg["seed"], cfg["dist"])
    rng = workloads.rng_for(1000)
    rows = [cfg["E"]] * cfg["T"]
    W, wo, Do = helpers.float_tables(rng, rows, [cfg["D"]] * cfg["T"], np.float32)
    want = oracle.tbe_forward(W, oracle.FP32, wo, Do, cfg["B"], inp.indices, inp.offsets)
    got, status = _run(W, wo, Do, rows, cfg["B"], inp.indices, inp.offsets, None, oracle.SUM,
                       torch.float32)
    assert status == 0
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=RTOL_FP32, atol=1e-7)


def test_forward_linearity_at_scale():
    """fp16 tables at a training-like size: pooling is linear in the per-sample weights, and a
    sampled set of bags matches the oracle."""
    T, E, D, B = 6, 200_000, 128, 4096
    inp = workloads.tbe_inputs(T, B, E, D, 1, 64, 2, "zipf", 1.05, permute=True)
    gen = torch.Generator(device="cuda").manual_seed(5)
    W = (torch.rand(T * E * D, device="cuda", generator=gen) * 0.02 - 0.01).half()
    wo = torch.arange(T, device="cuda", dtype=torch.int64) * (E * D)
    Do = torch.arange(T + 1, device="cuda", dtype=torch.int32) * D
    idx, off = _dev(inp.indices), _dev(inp.offsets)
    base = cabi.forward(W, wo, Do, T * D, D, idx, off, B)
    w1 = torch.rand(inp.num_lookups, device="cuda", generator=gen)
    a = cabi.forward(W, wo, Do, T * D, D, idx, off, B, per_sample_weights=w1)
    b = cabi.forward(W, wo, Do, T * D, D, idx, off, B, per_sample_weights=1.0 - w1)
    torch.testing.assert_close(a + b, base, rtol=1e-4, atol=1e-5)
    # sampled bags against the oracle: table 3, first 32 bags
    t = 3
    lo, hi = int(inp.offsets[t * B]), int(inp.offsets[t * B + 32])
    tab = W[t * E * D:(t + 1) * E * D].cpu().numpy()
    want = oracle.tbe_forward(tab, oracle.FP16, [0], [0, D], 32, inp.indices[lo:hi],
                              inp.offsets[t * B:t * B + 33] - lo)
    np.testing.assert_allclose(base[:32, t * D:(t + 1) * D].cpu().numpy(), want, rtol=RTOL_FP16,
                               atol=ATOL_FP16)
