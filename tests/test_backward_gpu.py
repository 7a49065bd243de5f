"""GPU parity: radix sort and the fused backward (exact SGD / row-wise Adagrad) vs the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle
from tests import helpers
from torchlib_xpu_b200 import cabi, workloads

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-3, 1e-3   # post-update weights (north-star tolerance)


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("n,key_dtype,bits", [
    (1, np.int32, 8), (31, np.int32, 5), (4096, np.int32, 13), (4097, np.int32, 25),
    (100_003, np.int32, 25), (1_000_000, np.int32, 28), (50_000, np.int64, 37), (8193, np.int64, 9),
    (300_000, np.int32, 32),
])
def test_radix_sort_is_a_stable_sort(n, key_dtype, bits):
    rng = workloads.rng_for(400 + n % 97)
    if bits <= 31:
        keys = rng.integers(0, 1 << bits, size=n, dtype=np.int64)
    else:
        keys = rng.integers(0, 1 << bits, size=n, dtype=np.uint64).astype(np.int64)
    if n > 1000:  # heavy repeats, as Zipf-distributed row ids give
        keys[rng.random(n) < 0.5] = keys[0]
    vals = np.arange(n, dtype=np.int32)
    ks, vs = cabi.radix_sort_pairs(_dev(keys.astype(key_dtype)), _dev(vals), bits)
    torch.cuda.synchronize()
    unsigned = keys.astype(np.uint64) & np.uint64((1 << bits) - 1)
    order = np.argsort(unsigned, kind="stable")
    want_k = keys.astype(key_dtype)[order]
    assert np.array_equal(ks.cpu().numpy(), want_k)
    assert np.array_equal(vs.cpu().numpy(), vals[order])


def test_radix_sort_ignores_high_bits():
    rng = workloads.rng_for(431)
    n, bits = 20_000, 10
    keys = rng.integers(0, 1 << 20, size=n, dtype=np.int64).astype(np.int32)
    vals = np.arange(n, dtype=np.int32)
    ks, vs = cabi.radix_sort_pairs(_dev(keys), _dev(vals), bits)
    order = np.argsort(keys & ((1 << bits) - 1), kind="stable")
    assert np.array_equal(ks.cpu().numpy(), keys[order])
    assert np.array_equal(vs.cpu().numpy(), vals[order])


@pytest.mark.parametrize("sizes,bits", [
    ([0, 5, 0, 4096, 4097, 1], 9), ([10_000, 300, 256, 257, 8192], 3), ([20_000, 9_000], 22),
    ([255, 256, 512, 1], 1), ([70_000], 11), ([3_000, 0, 0, 12_000, 0], 17), ([1] * 300, 5),
    ([150_000, 2, 90_000], 32),
])
@pytest.mark.parametrize("off_dtype", [np.int64, np.int32])
def test_segmented_sort_sorts_every_segment_on_its_own(sizes, bits, off_dtype):
    """b200tbe_radix_sort_segments (the backward's sort): every segment is stably sorted by the low
    bits of its keys, pairs never leave their segment; empty segments, segments that end inside a
    tile, one key per segment."""
    rng = workloads.rng_for(500 + len(sizes) + bits)
    n = int(sum(sizes))
    seg = np.zeros(len(sizes) + 1, dtype=np.int64)
    np.cumsum(sizes, out=seg[1:])
    keys = rng.integers(0, 1 << 32, size=n, dtype=np.uint64).astype(np.uint32)
    if n > 1000:
        keys[rng.random(n) < 0.4] = keys[0]
    vals = np.arange(n, dtype=np.int32)
    ks, vs = cabi.radix_sort_segments(_dev(keys.view(np.int32)), _dev(vals), _dev(seg.astype(off_dtype)), bits)
    torch.cuda.synchronize()
    want_k, want_v = np.empty_like(keys), np.empty_like(vals)
    mask = np.uint32((1 << bits) - 1) if bits < 32 else np.uint32(0xffffffff)
    for a, b in zip(seg[:-1], seg[1:]):
        order = np.argsort(keys[a:b] & mask, kind="stable")
        want_k[a:b], want_v[a:b] = keys[a:b][order], vals[a:b][order]
    assert np.array_equal(ks.cpu().numpy().view(np.uint32), want_k)
    assert np.array_equal(vs.cpu().numpy(), want_v)


def _backward_case(rng, rows, Ds, B, L_lo, L_hi, wdtype, gdtype, pooling, opt, weighted,
                   idx_dtype=np.int64, hot_row=None):
    T = len(Ds)
    W, wo, Do = helpers.float_tables(rng, rows, Ds, wdtype, -0.5, 0.5)
    _, offsets, indices = helpers.ragged_bags(rng, T, B, rows, L_lo, L_hi, empty_fraction=0.1)
    if hot_row is not None:  # one row drawn by most lookups of table 0: a long run
        a, b = int(offsets[0]), int(offsets[B])
        hot = rng.random(b - a) < 0.8
        indices[a:b][hot] = hot_row
    psw = rng.random(indices.size).astype(np.float32) if weighted else None
    total_D = int(Do[-1])
    grad = rng.standard_normal((B, total_D)).astype(np.float32)
    if gdtype == np.float16:
        grad = grad.astype(np.float16).astype(np.float32)
    hs = np.zeros(T + 1, dtype=np.int64)
    np.cumsum(np.asarray(rows, dtype=np.int64), out=hs[1:])
    mom = (rng.random(int(hs[-1])) * 0.1).astype(np.float32)
    return T, W, wo, Do, offsets, indices, psw, grad, hs, mom


def _check(T, W, wo, Do, offsets, indices, psw, grad, hs, mom, B, wdtype, gdtype, pooling, opt,
           idx_dtype=np.int64, lr=0.05, eps=1e-8, rows_hint=True, update_rtol=None):
    ty = oracle.FP32 if wdtype == np.float32 else oracle.FP16
    W_ref, m_ref = W.copy(), mom.copy()
    oracle.tbe_backward(W_ref, ty, wo, Do, hs, B, indices, offsets, grad, m_ref, hs[:-1], opt, lr, eps,
                        psw, pooling)
    bits = max(1, int(hs[-1] - 1).bit_length())
    dW, dm = _dev(W), _dev(mom)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    dgrad = _dev(grad.astype(gdtype))
    cabi.backward(dW, _dev(wo), _dev(Do), _dev(hs), bits, int(np.max(np.diff(Do))),
                  _dev(indices.astype(idx_dtype)), _dev(offsets.astype(idx_dtype)), B, dgrad, opt, lr,
                  eps, dm, _dev(hs[:-1].copy()), pooling, None if psw is None else _dev(psw),
                  status=status, max_table_rows=int(np.max(np.diff(hs))) if rows_hint else 0)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got_W = dW.float().cpu().numpy()
    np.testing.assert_allclose(got_W, W_ref.astype(np.float32), rtol=RTOL, atol=ATOL)
    if update_rtol is not None:
        # the absolute tolerance above is loose against small weights: compare the UPDATES too
        # (an fp16 row can only move in steps of its own spacing, hence the atol of two spacings)
        old = W.astype(np.float32)
        spacing = np.spacing(np.abs(W_ref).astype(np.float16)).astype(np.float32) if wdtype == np.float16 else 0.0
        np.testing.assert_allclose(got_W - old, W_ref.astype(np.float32) - old, rtol=update_rtol,
                                   atol=2 * np.max(spacing) + 1e-7)
    # rows that no lookup touched are bit-identical
    touched = np.zeros(int(hs[-1]), dtype=bool)
    for t in range(T):
        a, b = int(offsets[t * B]), int(offsets[(t + 1) * B])
        touched[hs[t] + np.unique(indices[a:b])] = True
    for t in range(T):
        D = int(Do[t + 1] - Do[t])
        tab_new = dW[wo[t]:wo[t] + (hs[t + 1] - hs[t]) * D].cpu().numpy().reshape(-1, D)
        tab_old = W[wo[t]:wo[t] + (hs[t + 1] - hs[t]) * D].reshape(-1, D)
        same = ~touched[hs[t]:hs[t + 1]]
        assert np.array_equal(tab_new[same].view(np.uint8), tab_old[same].view(np.uint8))
    if opt == oracle.ROWWISE_ADAGRAD:
        np.testing.assert_allclose(dm.cpu().numpy(), m_ref, rtol=1e-4, atol=1e-6)
    else:
        assert np.array_equal(dm.cpu().numpy(), mom)


@pytest.mark.parametrize("wdtype", [np.float32, np.float16])
@pytest.mark.parametrize("opt", [oracle.SGD, oracle.ROWWISE_ADAGRAD])
@pytest.mark.parametrize("pooling", [oracle.SUM, oracle.MEAN])
@pytest.mark.parametrize("weighted", [False, True])
def test_backward_mixed_dims(wdtype, opt, pooling, weighted):
    rng = workloads.rng_for(440)
    rows, Ds, B = [400, 90, 33, 700, 50], [128, 64, 8, 32, 256], 53
    case = _backward_case(rng, rows, Ds, B, 0, 30, wdtype, np.float32, pooling, opt, weighted)
    _check(*case, B, wdtype, np.float32, pooling, opt)


@pytest.mark.parametrize("gdtype", [np.float32, np.float16])
def test_backward_long_runs_and_fp16_grads(gdtype):
    """One row receives ~80% of a table's lookups: thousands of lookups in one run, which takes
    the chunked path."""
    rng = workloads.rng_for(441)
    rows, Ds, B = [1000, 64], [128, 64], 600
    case = _backward_case(rng, rows, Ds, B, 5, 40, np.float16, gdtype, oracle.SUM,
                          oracle.ROWWISE_ADAGRAD, False, hot_row=17)
    _check(*case, B, np.float16, gdtype, oracle.SUM, oracle.ROWWISE_ADAGRAD, lr=0.01)


@pytest.mark.parametrize("wdtype", [np.float32, np.float16])
def test_backward_wide_rows_with_fp16_gradients(wdtype):
    """Rows of 512 and 1024 elements with fp16 gradients (the 1024-element table runs on the ring
    engine, whose lanes hold elements, not gradient bytes), one of them with a long run."""
    rng = workloads.rng_for(444)
    rows, Ds, B = [300, 64], [512, 1024], 400
    case = _backward_case(rng, rows, Ds, B, 0, 12, wdtype, np.float16, oracle.SUM,
                          oracle.ROWWISE_ADAGRAD, False, hot_row=5)
    _check(*case, B, wdtype, np.float16, oracle.SUM, oracle.ROWWISE_ADAGRAD, lr=0.01)


@pytest.mark.parametrize("gdtype", [np.float32, np.float16])
@pytest.mark.parametrize("rows_hint", [True, False])
def test_backward_many_tables_runs_across_spans_and_tiles(gdtype, rows_hint):
    """Thirty tables of very different sizes (some without a lookup), two with a row that takes most of
    the table's lookups: runs of tens of thousands of lookups crossing spans and tiles of the plan,
    next to thousands of single-lookup runs. With and without the caller's bound on rows per table."""
    rng = workloads.rng_for(445)
    T, B = 30, 900
    rows = [int(r) for r in rng.integers(1, 3000, size=T)]
    Ds = [int(d) for d in rng.choice([4, 8, 16, 32, 64, 100, 128], size=T)]
    Ds[-1] += (-sum(Ds)) % 8                  # rows of the fp16 gradient matrix are whole 16-byte vectors
    W, wo, Do = helpers.float_tables(rng, rows, Ds, np.float16, -0.5, 0.5)
    lengths = rng.integers(0, 60, size=T * B, dtype=np.int64)
    for t in (3, 4, 17):                       # tables nobody looks up
        lengths[t * B:(t + 1) * B] = 0
    offsets = np.zeros(T * B + 1, dtype=np.int64)
    np.cumsum(lengths, out=offsets[1:])
    indices = np.zeros(int(offsets[-1]), dtype=np.int64)
    for t in range(T):
        a, b = int(offsets[t * B]), int(offsets[(t + 1) * B])
        indices[a:b] = rng.integers(0, rows[t], size=b - a)
        if t in (0, 11):
            indices[a:b][rng.random(b - a) < 0.85] = rows[t] // 2
    grad = rng.standard_normal((B, int(Do[-1]))).astype(np.float32)
    if gdtype == np.float16:
        grad = grad.astype(np.float16).astype(np.float32)
    hs = np.zeros(T + 1, dtype=np.int64)
    np.cumsum(np.asarray(rows, dtype=np.int64), out=hs[1:])
    mom = (rng.random(int(hs[-1])) * 0.1).astype(np.float32)
    _check(T, W, wo, Do, offsets, indices, None, grad, hs, mom, B, np.float16, gdtype, oracle.SUM,
           oracle.ROWWISE_ADAGRAD, lr=0.01, rows_hint=rows_hint)


def test_backward_run_of_only_bad_indices_leaves_row_zero_alone():
    """Out-of-range ids are filed under row 0 of their table; when row 0 has no valid lookup it must
    not be touched (with eps = 0 and zero state a zero gradient would otherwise divide by zero)."""
    rng = workloads.rng_for(446)
    rows, Ds, B = [50, 20], [64, 32], 12
    T, W, wo, Do, offsets, indices, psw, grad, hs, mom = _backward_case(
        rng, rows, Ds, B, 2, 6, np.float32, np.float32, oracle.SUM, oracle.ROWWISE_ADAGRAD, False)
    mom[:] = 0
    a, b = int(offsets[0]), int(offsets[B])
    indices[a:b][indices[a:b] == 0] = 1          # nobody looks up row 0 of table 0 ...
    indices[a + 3] = 1                            # (row 1 keeps at least one valid lookup)
    bad = indices.copy()
    bad[a:a + 3] = [50, 77, -1]                   # ... except three ids that are out of range
    keep = np.ones(indices.size, dtype=np.float32)
    keep[a:a + 3] = 0
    W_ref, m_ref = W.copy(), mom.copy()
    oracle.tbe_backward(W_ref, oracle.FP32, wo, Do, hs, B, np.where(keep > 0, indices, 1), offsets,
                        grad, m_ref, hs[:-1], oracle.ROWWISE_ADAGRAD, 0.1, 0.0, keep)
    dW, dm = _dev(W), _dev(mom)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cabi.backward(dW, _dev(wo), _dev(Do), _dev(hs), 7, 64, _dev(bad), _dev(offsets), B, _dev(grad),
                  oracle.ROWWISE_ADAGRAD, 0.1, 0.0, dm, _dev(hs[:-1].copy()), status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & cabi.DEV_INDEX_OUT_OF_RANGE
    got = dW.cpu().numpy()
    assert np.array_equal(got[:64].view(np.uint32), W[:64].view(np.uint32))   # row 0 of table 0: untouched
    assert np.isfinite(got).all() and float(dm[0].item()) == 0.0
    np.testing.assert_allclose(got, W_ref, rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(dm.cpu().numpy(), m_ref, rtol=1e-4, atol=1e-7)


def test_backward_int32_indices_wide_rows():
    rng = workloads.rng_for(442)
    rows, Ds, B = [64, 40], [512, 1024], 21
    case = _backward_case(rng, rows, Ds, B, 0, 12, np.float32, np.float32, oracle.MEAN,
                          oracle.ROWWISE_ADAGRAD, True)
    _check(*case, B, np.float32, np.float32, oracle.MEAN, oracle.ROWWISE_ADAGRAD, idx_dtype=np.int32)


def test_backward_flags_bad_indices_and_skips_them():
    rng = workloads.rng_for(443)
    rows, Ds, B = [50], [64], 10
    T, W, wo, Do, offsets, indices, psw, grad, hs, mom = _backward_case(
        rng, rows, Ds, B, 2, 6, np.float32, np.float32, oracle.SUM, oracle.SGD, False)
    bad = indices.copy()
    bad[2] = 50
    keep = np.ones(indices.size, dtype=np.float32)
    keep[2] = 0
    W_ref = W.copy()
    oracle.tbe_backward(W_ref, oracle.FP32, wo, Do, hs, B, np.where(keep > 0, indices, 0), offsets,
                        grad, None, None, oracle.SGD, 0.1, 0.0, keep)
    dW = _dev(W)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cabi.backward(dW, _dev(wo), _dev(Do), _dev(hs), 6, 64, _dev(bad), _dev(offsets), B, _dev(grad),
                  oracle.SGD, 0.1, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & cabi.DEV_INDEX_OUT_OF_RANGE
    np.testing.assert_allclose(dW.cpu().numpy(), W_ref, rtol=1e-5, atol=1e-6)


def test_backward_named_training_config_scaled_down():
    """The training configuration's shape (fp16 tables, fp32 state and gradients, Zipf(1.05) ids
    through a fixed permutation, L~U{1..64}, lr 0.01, eps 1e-8) with fewer and smaller tables."""
    T, E, D, B = 4, 100_000, 128, 2048
    inp = workloads.tbe_inputs(T, B, E, D, 1, 64, 2, "zipf", 1.05, permute=True)
    rng = workloads.rng_for(2000)
    W, wo, Do = helpers.float_tables(rng, [E] * T, [D] * T, np.float16, -0.01, 0.01)
    hs = np.arange(T + 1, dtype=np.int64) * E
    grad = rng.standard_normal((B, T * D)).astype(np.float32)
    mom = np.zeros(T * E, dtype=np.float32)
    _check(T, W, wo, Do, inp.offsets, inp.indices, None, grad, hs, mom, B, np.float16, np.float32,
           oracle.SUM, oracle.ROWWISE_ADAGRAD, lr=0.01, update_rtol=1e-2)


def test_backward_waits_for_the_gradient_event():
    """grad_ready_event: the gradient matrix is produced on another stream, after a long kernel; the
    backward started before it is complete still updates with the complete gradients."""
    rng = workloads.rng_for(470)
    B = 64
    case = _backward_case(rng, [300, 200], [64, 128], B, 0, 12, np.float16, np.float32, oracle.SUM,
                          oracle.ROWWISE_ADAGRAD, False)
    T, W, wo, Do, offsets, indices, psw, grad, hs, mom = case
    W_ref, m_ref = W.copy(), mom.copy()
    oracle.tbe_backward(W_ref, oracle.FP16, wo, Do, hs, B, indices, offsets, grad, m_ref, hs[:-1],
                        oracle.ROWWISE_ADAGRAD, 0.05, 1e-8, None, oracle.SUM)
    dW, dm = _dev(W), _dev(mom)
    src = _dev(grad)
    dgrad = torch.zeros_like(src)            # wrong until the side stream has written it
    filler = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    side = torch.cuda.Stream()
    ready = torch.cuda.Event()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        for _ in range(20):                  # a few milliseconds of work ahead of the gradient copy
            filler.zero_()
        dgrad.copy_(src)
        ready.record(side)
    bits = max(1, int(hs[-1] - 1).bit_length())
    cabi.backward(dW, _dev(wo), _dev(Do), _dev(hs), bits, 128, _dev(indices), _dev(offsets), B, dgrad,
                  oracle.ROWWISE_ADAGRAD, 0.05, 1e-8, dm, _dev(hs[:-1].copy()), grad_ready_event=ready)
    torch.cuda.synchronize()
    np.testing.assert_allclose(dW.float().cpu().numpy(), W_ref.astype(np.float32), rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(dm.cpu().numpy(), m_ref, rtol=1e-4, atol=1e-6)
