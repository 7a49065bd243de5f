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
           idx_dtype=np.int64, lr=0.05, eps=1e-8):
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
                  status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got_W = dW.float().cpu().numpy()
    np.testing.assert_allclose(got_W, W_ref.astype(np.float32), rtol=RTOL, atol=ATOL)
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
           oracle.SUM, oracle.ROWWISE_ADAGRAD, lr=0.01)


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
