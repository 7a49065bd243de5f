"""Pins the C oracle (oracle/tbe_oracle.c) against independent CPU implementations:
FBGEMM-core kernels bundled in torch's libtorch_cpu.so, ATen CPU ops and naive Python loops.
No GPU needed."""
import numpy as np
import pytest
import torch

import oracle
from tests import helpers
from torchlib_xpu_b200 import workloads


def test_half_conversions_match_numpy():
    lib = oracle.c_lib()
    halves = np.arange(65536, dtype=np.uint16)
    want = halves.view(np.float16).astype(np.float32)
    got = np.array([lib.oracle_half_to_float(int(h)) for h in halves], dtype=np.float32)
    nan = np.isnan(want)  # NaN payloads may be quieted on the way through the C return value
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan])
    rng = workloads.rng_for(7)
    xs = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 20000),
        halves.view(np.float16).astype(np.float32)[::17],
        np.array([65504.0, 65519.9, 65520.0, 1e-8, 2.98e-8, 2.99e-8, 5.96e-8, 6.1e-5, 0.0, -0.0],
                 dtype=np.float32),
    ]).astype(np.float32)
    xs = xs[np.isfinite(xs)]
    with np.errstate(over="ignore"):
        want_h = xs.astype(np.float16).view(np.uint16)
    got_h = np.array([lib.oracle_float_to_half(float(x)) for x in xs], dtype=np.uint16)
    assert np.array_equal(got_h, want_h)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("pooling", [oracle.SUM, oracle.MEAN])
@pytest.mark.parametrize("weighted", [False, True])
def test_forward_matches_fbgemm_core_and_embedding_bag(dtype, pooling, weighted):
    rng = workloads.rng_for(11)
    rows, Ds, B = [50, 300, 7], [128, 64, 20], 37
    T = len(Ds)
    W, wo, Do = helpers.float_tables(rng, rows, Ds, dtype)
    _, offsets, indices = helpers.ragged_bags(rng, T, B, rows, 0, 9, empty_fraction=0.2)
    psw = rng.random(indices.size).astype(np.float32) if weighted else None
    ty = oracle.FP32 if dtype == np.float32 else oracle.FP16
    got = oracle.tbe_forward(W, ty, wo, Do, B, indices, offsets, psw, pooling, backend="c")
    ref = oracle.tbe_forward(W, ty, wo, Do, B, indices, offsets, psw, pooling, backend="ref",
                             rows_per_table=rows)
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-7)
    if weighted and pooling == oracle.MEAN:
        return  # embedding_bag has no weighted mean
    for t in range(T):
        tab = torch.from_numpy(W[wo[t]:wo[t] + rows[t] * Ds[t]].astype(np.float32).reshape(rows[t], Ds[t]))
        off_t = offsets[t * B:(t + 1) * B + 1]
        idx_t = torch.from_numpy(indices[off_t[0]:off_t[-1]])
        eb = torch.nn.functional.embedding_bag(
            idx_t, tab, torch.from_numpy(off_t - off_t[0]), mode="sum" if (pooling == oracle.SUM) else "mean",
            per_sample_weights=None if psw is None else torch.from_numpy(psw[off_t[0]:off_t[-1]]),
            include_last_offset=True)
        np.testing.assert_allclose(got[:, Do[t]:Do[t + 1]], eb.numpy(), rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("row_alignment", [16, 1])
@pytest.mark.parametrize("pooling", [oracle.SUM, oracle.MEAN])
def test_nbit_forward_matches_fbgemm_core(row_alignment, pooling):
    rng = workloads.rng_for(12)
    tys = [oracle.INT8, oracle.INT4, oracle.INT2, oracle.FP16, oracle.FP32, oracle.INT4]
    Ds = [128, 128, 64, 32, 16, 40]
    rows = [40, 33, 21, 10, 9, 17]
    T, B = len(tys), 29
    W, wo, Do, tys_a = helpers.quantised_tables(rng, rows, Ds, tys, row_alignment)
    _, offsets, indices = helpers.ragged_bags(rng, T, B, rows, 0, 12, empty_fraction=0.15)
    psw = rng.random(indices.size).astype(np.float32)
    for w in (None, psw):
        got = oracle.nbit_forward(W, wo, tys_a, Do, row_alignment, B, indices, offsets, w, pooling)
        ref = oracle.nbit_forward(W, wo, tys_a, Do, row_alignment, B, indices, offsets, w, pooling,
                                  backend="ref", rows_per_table=rows)
        np.testing.assert_allclose(got, ref, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("ty,D", [(oracle.INT8, 128), (oracle.INT4, 128), (oracle.INT2, 64),
                                  (oracle.INT8, 20), (oracle.INT4, 36)])
def test_quantiser_matches_fbgemm_core(ty, D):
    rng = workloads.rng_for(13)
    src = rng.uniform(-1, 1, size=(257, D)).astype(np.float32)
    src[3] = 0.25  # constant row: zero range
    mine = oracle.quantize_rows(src, ty, 1, backend="c")
    ref = oracle.quantize_rows(src, ty, 1, backend="ref")
    # headers (fp16 scale, bias) must agree exactly; payload may differ by one step on ties
    assert np.array_equal(mine[:, :4], ref[:, :4])
    bits = {oracle.INT8: 8, oracle.INT4: 4, oracle.INT2: 2}[ty]
    deq_mine = oracle.dequantize_rows_ref(mine, D, ty)
    deq_ref = oracle.dequantize_rows_ref(ref, D, ty)
    scale = mine[:, :2].copy().view(np.float16).astype(np.float32)
    assert np.all(np.abs(deq_mine - deq_ref) <= scale * 1.001 + 1e-6)
    assert np.mean(mine == ref) > 0.995
    # and the dequantised values reproduce the source within one quantisation step
    assert np.all(np.abs(deq_mine - src) <= scale * (1.0 if bits < 8 else 1.0) + 2e-3)


@pytest.mark.parametrize("ty,D", [(oracle.INT8, 128), (oracle.INT4, 64), (oracle.INT2, 32)])
def test_nbit_element_matches_fbgemm_dequantise(ty, D):
    rng = workloads.rng_for(14)
    src = rng.uniform(-1, 1, size=(64, D)).astype(np.float32)
    rows = oracle.quantize_rows(src, ty, 1)
    want = oracle.dequantize_rows_ref(rows, D, ty)
    # one bag per row, SUM pooling == plain dequantisation
    n = rows.shape[0]
    got = oracle.nbit_forward(rows.reshape(-1), np.zeros(1, np.int64), np.array([ty], np.uint8),
                              np.array([0, D], np.int32), 1, n, np.arange(n), np.arange(n + 1))
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_rowwise_adagrad_formula_matches_fbgemm_core(dtype):
    """Without repeated rows the exact update equals FBGEMM-core's fused row-wise Adagrad."""
    rng = workloads.rng_for(15)
    rows, D, B = 500, 64, 40
    w0 = workloads.uniform_table(rng, rows, D, -0.1, 0.1, dtype)
    h0 = rng.random(rows).astype(np.float32) * 0.01
    perm = rng.permutation(rows)
    lengths = rng.integers(0, 6, size=B)
    offsets = np.zeros(B + 1, dtype=np.int64)
    np.cumsum(lengths, out=offsets[1:])
    indices = perm[:offsets[-1]].astype(np.int64)  # every row at most once
    grad = rng.standard_normal((B, D)).astype(np.float32)
    lr, eps = 0.01, 1e-8
    w_ref, h_ref = w0.copy(), h0.copy()
    oracle.rowwise_adagrad_fused_ref(w_ref, grad, h_ref, indices, offsets, eps, lr)
    w_mine, h_mine = w0.copy().reshape(-1), h0.copy()
    ty = oracle.FP32 if dtype == np.float32 else oracle.FP16
    oracle.tbe_backward(w_mine, ty, [0], [0, D], [0, rows], B, indices, offsets, grad, h_mine, [0],
                        oracle.ROWWISE_ADAGRAD, lr, eps)
    np.testing.assert_allclose(h_mine, h_ref, rtol=1e-6, atol=1e-9)
    tol = 1e-6 if dtype == np.float32 else 1e-3
    np.testing.assert_allclose(w_mine.reshape(rows, D).astype(np.float32), w_ref.astype(np.float32),
                               rtol=tol, atol=tol * 1e-2)
    assert not np.array_equal(w_mine.reshape(rows, D), w0)


def test_backward_exact_semantics_against_python_loop():
    """Repeated rows are summed first, then updated once (SGD and Adagrad, SUM and MEAN)."""
    rng = workloads.rng_for(16)
    rows, Ds, B = [30, 12], [8, 12], 25
    T = 2
    for pooling in (oracle.SUM, oracle.MEAN):
        for opt in (oracle.SGD, oracle.ROWWISE_ADAGRAD):
            W, wo, Do = helpers.float_tables(rng, rows, Ds, np.float32, -1, 1)
            _, offsets, indices = helpers.ragged_bags(rng, T, B, rows, 0, 8, 0.1)
            psw = rng.random(indices.size).astype(np.float32)
            grad = rng.standard_normal((B, int(Do[-1]))).astype(np.float32)
            hs = np.array([0, rows[0], rows[0] + rows[1]], dtype=np.int64)
            mom = rng.random(int(hs[-1])).astype(np.float32)
            W1, m1 = W.copy(), mom.copy()
            oracle.tbe_backward(W1, oracle.FP32, wo, Do, hs, B, indices, offsets, grad, m1, hs[:-1],
                                opt, 0.05, 1e-8, psw, pooling)
            W2, m2 = W.astype(np.float64), mom.astype(np.float64)
            for t in range(T):
                gsum = np.zeros((rows[t], Ds[t]))
                for b in range(B):
                    bag = t * B + b
                    L = offsets[bag + 1] - offsets[bag]
                    for j in range(offsets[bag], offsets[bag + 1]):
                        w = psw[j] / (L if pooling == oracle.MEAN else 1)
                        gsum[indices[j]] += grad[b, Do[t]:Do[t + 1]] * w
                touched = np.unique(indices[offsets[t * B]:offsets[(t + 1) * B]])
                for r in touched:
                    g = gsum[r]
                    mult = 0.05
                    if opt == oracle.ROWWISE_ADAGRAD:
                        m2[hs[t] + r] += np.mean(g * g)
                        mult = 0.05 / (np.sqrt(m2[hs[t] + r]) + 1e-8)
                    W2[wo[t] + r * Ds[t]: wo[t] + (r + 1) * Ds[t]] -= mult * g
            np.testing.assert_allclose(W1, W2, rtol=2e-5, atol=1e-6)
            if opt == oracle.ROWWISE_ADAGRAD:
                np.testing.assert_allclose(m1, m2, rtol=2e-5, atol=1e-7)
            else:
                assert np.array_equal(m1, mom)


@pytest.mark.parametrize("dtype", [np.float32, np.float16, np.int64, np.uint8])
def test_jagged_single_level_matches_aten(dtype):
    rng = workloads.rng_for(17)
    B, max_L, D = 23, 9, 6
    lengths = rng.integers(0, 14, size=B)  # some rows longer than max_L: truncated
    offsets = np.zeros(B + 1, dtype=np.int64)
    np.cumsum(lengths, out=offsets[1:])
    if np.issubdtype(dtype, np.floating):
        values = rng.standard_normal((offsets[-1], D)).astype(dtype)
    else:
        values = rng.integers(0, 200, size=(offsets[-1], D)).astype(dtype)
    dense = oracle.jagged_to_padded_dense(values, [offsets], [max_L], 3)
    tv, to = torch.from_numpy(values), torch.from_numpy(offsets)
    want = torch.ops.aten._jagged_to_padded_dense_forward(tv, [to], [max_L], 3.0)
    assert np.array_equal(dense.view(np.uint8), want.numpy().view(np.uint8))
    # ATen's inverse rejects lengths above max_L; ours defines those rows as zero
    back = oracle.dense_to_jagged(dense, [offsets], int(offsets[-1]))
    l_of = np.concatenate([np.arange(n) for n in lengths])
    inside = l_of < max_L
    assert np.array_equal(back[inside], values[inside])
    assert np.all(back[~inside] == 0)
    # lengths within max_L: the inverse agrees with ATen's
    lengths2 = np.minimum(lengths, max_L)
    offsets2 = np.zeros(B + 1, dtype=np.int64)
    np.cumsum(lengths2, out=offsets2[1:])
    to2 = torch.from_numpy(offsets2)
    back2 = oracle.dense_to_jagged(dense, [offsets2], int(offsets2[-1]))
    want_back2 = torch.ops.aten._padded_dense_to_jagged_forward(want, [to2], int(offsets2[-1]))
    assert np.array_equal(back2.view(np.uint8), want_back2.numpy().view(np.uint8))


def _naive_to_dense(values, offsets_list, max_lengths, pad):
    outer = len(offsets_list[0]) - 1
    inner = values.shape[1]
    dense = np.full((outer, *max_lengths, inner), pad, dtype=values.dtype)
    for pos in np.ndindex(outer, *max_lengths):
        idx, ok = pos[0], True
        for d, off in enumerate(offsets_list):
            begin, end = off[idx], off[idx + 1]
            if pos[d + 1] >= end - begin:
                ok = False
                break
            idx = begin + pos[d + 1]
        if ok:
            dense[pos] = values[idx]
    return dense


def test_jagged_nested_levels_match_python_loop():
    rng = workloads.rng_for(18)
    outer = 5
    l1 = rng.integers(0, 5, size=outer)
    o1 = np.zeros(outer + 1, dtype=np.int64)
    np.cumsum(l1, out=o1[1:])
    l2 = rng.integers(0, 6, size=o1[-1])
    o2 = np.zeros(o1[-1] + 1, dtype=np.int64)
    np.cumsum(l2, out=o2[1:])
    values = rng.standard_normal((o2[-1], 3)).astype(np.float32)
    max_lengths = [3, 4]
    dense = oracle.jagged_to_padded_dense(values, [o1, o2], max_lengths, -1.5)
    want = _naive_to_dense(values, [o1, o2], max_lengths, np.float32(-1.5))
    assert np.array_equal(dense, want)
    y = rng.standard_normal(dense.shape).astype(np.float32)
    added = oracle.jagged_dense_elementwise_add(values, [o1, o2], y)
    assert np.array_equal(added, _naive_to_dense(values, [o1, o2], max_lengths, np.float32(0)) + y)
    back = oracle.dense_to_jagged(want, [o1, o2], int(o2[-1]))
    again = oracle.jagged_to_padded_dense(back, [o1, o2], max_lengths, -1.5)
    assert np.array_equal(again, want)


def test_jagged_add_matches_aten_plus_y():
    rng = workloads.rng_for(19)
    j = workloads.jagged_inputs(64, 16, 32, 19)
    x = rng.standard_normal((j.total_rows, j.D)).astype(np.float32)
    y = rng.standard_normal((j.B, j.max_L, j.D)).astype(np.float32)
    got = oracle.jagged_dense_elementwise_add(x, [j.offsets], y)
    want = torch.ops.aten._jagged_to_padded_dense_forward(
        torch.from_numpy(x), [torch.from_numpy(j.offsets)], [j.max_L], 0.0) + torch.from_numpy(y)
    assert np.array_equal(got, want.numpy())
