"""GPU parity through the drop-in boundary: torch.ops.fbgemm.* (the C++ operator library, which
calls the C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle
from tests import helpers
import torchlib_xpu_b200
from torchlib_xpu_b200 import workloads

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _ops():
    torchlib_xpu_b200.load_torch_ops()


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_jagged_ops_match_oracle_bit_for_bit():
    j = workloads.jagged_inputs(128, 24, 64, 1)
    rng = workloads.rng_for(501)
    values = rng.standard_normal((j.total_rows, j.D)).astype(np.float32)
    y = rng.standard_normal((j.B, j.max_L, j.D)).astype(np.float32)
    off = _dev(j.offsets)
    dense = torch.ops.fbgemm.jagged_to_padded_dense(_dev(values), [off], [j.max_L], 0.5)
    want = oracle.jagged_to_padded_dense(values, [j.offsets], [j.max_L], 0.5)
    assert np.array_equal(dense.cpu().numpy(), want)
    back, offs = torch.ops.fbgemm.dense_to_jagged(dense, [off], j.total_rows)
    assert np.array_equal(back.cpu().numpy(), values) and offs[0] is not None
    back2, _ = torch.ops.fbgemm.dense_to_jagged(dense, [off])
    assert torch.equal(back, back2)
    out = torch.ops.fbgemm.jagged_dense_elementwise_add(_dev(values), [off], _dev(y))
    assert np.array_equal(out.cpu().numpy(), oracle.jagged_dense_elementwise_add(values, [j.offsets], y))
    d2 = torch.ops.fbgemm.jagged_2d_to_dense(_dev(values), off, j.max_L)
    assert np.array_equal(d2.cpu().numpy(), oracle.jagged_to_padded_dense(values, [j.offsets], [j.max_L], 0))
    # 1-D values
    v1 = torch.ops.fbgemm.jagged_to_padded_dense(_dev(values[:, 0].copy()), [off], [j.max_L], 0.0)
    want1 = oracle.jagged_to_padded_dense(values[:, :1].copy(), [j.offsets], [j.max_L], 0)[..., 0]
    assert np.array_equal(v1.cpu().numpy(), want1)


def test_jagged_ops_are_differentiable():
    """Each copy's gradient is the other copy of the output gradient (bit-exact: the backward passes are
    the same kernels); the add hands its gradient to y unchanged and to x through dense_to_jagged."""
    j = workloads.jagged_inputs(96, 20, 32, 3)
    rng = workloads.rng_for(502)
    values = rng.standard_normal((j.total_rows, j.D)).astype(np.float32)
    y = rng.standard_normal((j.B, j.max_L, j.D)).astype(np.float32)
    w = rng.standard_normal((j.B, j.max_L, j.D)).astype(np.float32)
    wj = rng.standard_normal((j.total_rows, j.D)).astype(np.float32)
    off = _dev(j.offsets)

    v = _dev(values).requires_grad_(True)
    dense = torch.ops.fbgemm.jagged_to_padded_dense(v, [off], [j.max_L], 7.0)
    assert dense.grad_fn is not None
    (dense * _dev(w)).sum().backward()
    assert np.array_equal(v.grad.cpu().numpy(), oracle.dense_to_jagged(w, [j.offsets], j.total_rows))

    d = _dev(y).requires_grad_(True)
    back, _ = torch.ops.fbgemm.dense_to_jagged(d, [off], j.total_rows)
    (back * _dev(wj)).sum().backward()
    assert np.array_equal(d.grad.cpu().numpy(), oracle.jagged_to_padded_dense(wj, [j.offsets], [j.max_L], 0.0))

    x = _dev(values).requires_grad_(True)
    yy = _dev(y).requires_grad_(True)
    out = torch.ops.fbgemm.jagged_dense_elementwise_add(x, [off], yy)
    (out * _dev(w)).sum().backward()
    assert np.array_equal(yy.grad.cpu().numpy(), w)
    assert np.array_equal(x.grad.cpu().numpy(), oracle.dense_to_jagged(w, [j.offsets], j.total_rows))
    # no graph, no node
    assert torch.ops.fbgemm.jagged_to_padded_dense(_dev(values), [off], [j.max_L], 0.0).grad_fn is None


def test_device_status_word_reports_bad_ids_from_the_ops():
    """The lookup ops range-check ids against hash_size_cumsum; a bad id is skipped and shows up in
    torch.ops.fbgemm.b200tbe_pop_device_status, which clears the word."""
    T, E, D, B = 2, 50, 16, 4
    w = torch.ones(T * E * D, device="cuda")
    wo = torch.arange(T, device="cuda", dtype=torch.int64) * (E * D)
    Do = torch.arange(T + 1, device="cuda", dtype=torch.int32) * D
    hs = torch.arange(T + 1, device="cuda", dtype=torch.int64) * E
    offsets = torch.arange(T * B + 1, device="cuda", dtype=torch.int64) * 2
    idx = torch.randint(0, E, (T * B * 2,), device="cuda")
    e, ei = _empty(), _empty(torch.int32)
    args = lambda ids: (torch.zeros(1, device="cuda"), w, e, e, ei, wo, Do, T * D, D, hs, 7, ids, offsets, 0, None,
                        None, ei, False, 0.0, False, 0.0, 0)
    torch.ops.fbgemm.b200tbe_pop_device_status(w)
    out = torch.ops.fbgemm.split_embedding_codegen_lookup_sgd_function(*args(idx))
    assert torch.ops.fbgemm.b200tbe_pop_device_status(w) == 0
    assert torch.equal(out, torch.full((B, T * D), 2.0, device="cuda"))
    bad = idx.clone()
    bad[3] = E                       # one row past the table
    out = torch.ops.fbgemm.split_embedding_codegen_lookup_sgd_function(*args(bad))
    assert torch.ops.fbgemm.b200tbe_pop_device_status(w) & 1      # B200TBE_DEV_INDEX_OUT_OF_RANGE
    assert torch.ops.fbgemm.b200tbe_pop_device_status(w) == 0     # popped
    assert float(out[1, :D].sum()) == D                           # the bad lookup was skipped, its neighbour pooled


def test_ops_reject_cpu_tensors_and_bad_shapes():
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.fbgemm.jagged_to_padded_dense(torch.zeros(3, 2), [torch.zeros(2, dtype=torch.int64)], [2], 0.0)
    off = torch.zeros(3, dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError):
        torch.ops.fbgemm.jagged_dense_elementwise_add(
            torch.zeros(0, 4, device="cuda"), [off], torch.zeros(2, 3, 5, device="cuda"))


def _empty(dtype=torch.float32):
    return torch.empty(0, dtype=dtype, device="cuda")


@pytest.mark.parametrize("optimizer", ["sgd", "rowwise_adagrad"])
@pytest.mark.parametrize("wdtype", [np.float32, np.float16])
def test_training_lookup_forward_and_fused_backward(optimizer, wdtype):
    rng = workloads.rng_for(502)
    rows, Ds, B = [300, 80, 500], [128, 32, 64], 96
    T = len(Ds)
    W, wo, Do = helpers.float_tables(rng, rows, Ds, wdtype, -0.1, 0.1)
    _, offsets, indices = helpers.ragged_bags(rng, T, B, rows, 0, 20, 0.1)
    hs = np.zeros(T + 1, dtype=np.int64)
    np.cumsum(np.asarray(rows, dtype=np.int64), out=hs[1:])
    bits = int(hs[-1] - 1).bit_length()
    mom = (rng.random(int(hs[-1])) * 0.05).astype(np.float32)
    grad = rng.standard_normal((B, int(Do[-1]))).astype(np.float32)
    ty = oracle.FP32 if wdtype == np.float32 else oracle.FP16

    dW, dm = _dev(W), _dev(mom)
    placeholder = torch.zeros(1, device="cuda", requires_grad=True)
    common = (placeholder, dW, _empty(dW.dtype), _empty(dW.dtype), _empty(torch.int32), _dev(wo), _dev(Do),
              int(Do[-1]), max(Ds), _dev(hs), bits, _dev(indices), _dev(offsets), 0, None, None,
              _empty(torch.int32), False, 0.0, False)
    if optimizer == "sgd":
        out = torch.ops.fbgemm.split_embedding_codegen_lookup_sgd_function(*common, 0.05, 0)
    else:
        out = torch.ops.fbgemm.split_embedding_codegen_lookup_rowwise_adagrad_function(
            *common, dm, _empty(), _empty(torch.int32), _dev(hs[:-1].copy()), 1e-8, 0.05)
    want = oracle.tbe_forward(W, ty, wo, Do, B, indices, offsets)
    tol = dict(rtol=1e-5, atol=5e-6) if wdtype == np.float32 else dict(rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(out.detach().cpu().numpy(), want, **tol)

    out.backward(_dev(grad))
    torch.cuda.synchronize()
    W_ref, m_ref = W.copy(), mom.copy()
    oracle.tbe_backward(W_ref, ty, wo, Do, hs, B, indices, offsets, grad, m_ref, hs[:-1],
                        oracle.SGD if optimizer == "sgd" else oracle.ROWWISE_ADAGRAD, 0.05, 1e-8)
    np.testing.assert_allclose(dW.float().cpu().numpy(), W_ref.astype(np.float32), rtol=1e-3, atol=1e-3)
    assert not np.array_equal(dW.cpu().numpy(), W)
    if optimizer == "rowwise_adagrad":
        np.testing.assert_allclose(dm.cpu().numpy(), m_ref, rtol=1e-4, atol=1e-6)
    assert placeholder.grad is None or float(placeholder.grad.abs().sum()) == 0.0


def test_training_lookup_rejects_unsupported_features():
    z = torch.zeros(2, dtype=torch.int64, device="cuda")
    args = [torch.zeros(1, device="cuda", requires_grad=True), torch.zeros(8, device="cuda"), _empty(), _empty(),
            _empty(torch.int32), torch.zeros(1, dtype=torch.int64, device="cuda"),
            torch.tensor([0, 4], dtype=torch.int32, device="cuda"), 4, 4, z, 1, z[:0], z[:2], 0, None,
            None, _empty(torch.int32), False, 0.0, True]  # stochastic_rounding=True
    with pytest.raises(RuntimeError, match="stochastic_rounding"):
        torch.ops.fbgemm.split_embedding_codegen_lookup_sgd_function(*args, 0.1, 0)


def test_nbit_lookup_op():
    rng = workloads.rng_for(503)
    tys = [oracle.INT8, oracle.INT4, oracle.FP16]
    Ds, rows, B = [128, 128, 64], [200, 150, 40], 64
    W, wo, Do, tys_a = helpers.quantised_tables(rng, rows, Ds, tys, 16)
    _, offsets, indices = helpers.ragged_bags(rng, 3, B, rows, 0, 30, 0.1)
    out = torch.ops.fbgemm.int_nbit_split_embedding_codegen_lookup_function(
        _dev(W), torch.empty(0, dtype=torch.uint8, device="cuda"), _empty(torch.int32), _dev(wo),
        _dev(tys_a), _dev(Do), int(Do[-1]), 0, 128, 128, 64, 0, _dev(indices), _dev(offsets), 0, None, 1,
        None, None, 16)
    assert out.dtype == torch.float16
    want = oracle.nbit_forward(W, wo, tys_a, Do, 16, B, indices, offsets)
    np.testing.assert_allclose(out.float().cpu().numpy(), want, rtol=1e-3, atol=1e-3)


def test_permute_2d_sparse_data_rows_may_repeat_or_drop():
    """torch.ops.fbgemm.permute_2D_sparse_data: row j of the result is row permute[j] of the input."""
    rng = workloads.rng_for(1400)
    T, B = 6, 37
    lengths = rng.integers(0, 9, size=(T, B)).astype(np.int64)
    total = int(lengths.sum())
    indices = rng.integers(0, 1 << 40, size=total, dtype=np.int64)
    weights = rng.standard_normal(total).astype(np.float32)
    permute = np.array([4, 0, 0, 5, 2], dtype=np.int32)      # row 0 twice, rows 1 and 3 dropped
    row_start = np.concatenate([[0], np.cumsum(lengths.sum(1))])
    want_idx = np.concatenate([indices[row_start[t]:row_start[t + 1]] for t in permute])
    want_w = np.concatenate([weights[row_start[t]:row_start[t + 1]] for t in permute])
    dev = lambda a: torch.from_numpy(a).cuda()
    pl, pi, pw = torch.ops.fbgemm.permute_2D_sparse_data(dev(permute), dev(lengths), dev(indices), dev(weights), None)
    assert np.array_equal(pl.cpu().numpy(), lengths[permute])
    assert np.array_equal(pi.cpu().numpy(), want_idx)
    assert np.array_equal(pw.cpu().numpy(), want_w)
    pl2, pi2, none = torch.ops.fbgemm.permute_2D_sparse_data(dev(permute.astype(np.int64)), dev(lengths.astype(np.int32)),
                                                             dev(indices.astype(np.int32)), None, int(want_idx.size))
    assert none is None and np.array_equal(pi2.cpu().numpy(), want_idx.astype(np.int32))
    assert np.array_equal(pl2.cpu().numpy(), lengths[permute].astype(np.int32))
