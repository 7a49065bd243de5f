"""GPU parity of the module facades (the callers one step above the operator boundary)."""
import numpy as np
import pytest
import torch

import oracle
from tests import helpers
from torchlib_xpu_b200 import workloads
from torchlib_xpu_b200.tbe_modules import (IntNBitTableBatchedEmbeddingBagsCodegen, OptimType, PoolingMode,
                                           SparseType, SplitTableBatchedEmbeddingBagsCodegen)

pytestmark = pytest.mark.gpu


def test_training_module_steps_match_the_oracle():
    rng = workloads.rng_for(700)
    specs, B = [(500, 128), (300, 64), (80, 32)], 64
    mod = SplitTableBatchedEmbeddingBagsCodegen(specs, OptimType.EXACT_ROWWISE_ADAGRAD, 0.05, 1e-8,
                                                PoolingMode.MEAN, SparseType.FP16)
    W = mod.weights_dev.detach().cpu().numpy().copy()
    mom = np.zeros(sum(r for r, _ in specs), dtype=np.float32)
    wo = mod.weights_offsets.cpu().numpy()
    Do = mod.D_offsets.cpu().numpy()
    hs = mod.hash_size_cumsum.cpu().numpy()
    for step in range(2):
        _, offsets, indices = helpers.ragged_bags(rng, len(specs), B, [r for r, _ in specs], 0, 12, 0.1)
        grad = rng.standard_normal((B, int(Do[-1]))).astype(np.float32)
        out = mod(torch.from_numpy(indices).cuda(), torch.from_numpy(offsets).cuda())
        want = oracle.tbe_forward(W, oracle.FP16, wo, Do, B, indices, offsets, None, oracle.MEAN)
        np.testing.assert_allclose(out.detach().cpu().numpy(), want, rtol=1e-3, atol=1e-3)
        out.backward(torch.from_numpy(grad).cuda())
        oracle.tbe_backward(W, oracle.FP16, wo, Do, hs, B, indices, offsets, grad, mom, hs[:-1],
                            oracle.ROWWISE_ADAGRAD, 0.05, 1e-8, None, oracle.MEAN)
        torch.cuda.synchronize()
        np.testing.assert_allclose(mod.weights_dev.detach().float().cpu().numpy(), W.astype(np.float32),
                                   rtol=1e-3, atol=1e-3)
        np.testing.assert_allclose(mod.momentum1_dev.cpu().numpy(), mom, rtol=1e-4, atol=1e-6)
        W = mod.weights_dev.detach().cpu().numpy().copy()   # keep the two in lock step
        mom = mod.momentum1_dev.cpu().numpy().copy()
    views = mod.split_embedding_weights()
    assert [tuple(v.shape) for v in views] == specs


def test_inference_module_quantises_and_pools():
    rng = workloads.rng_for(701)
    specs = [(200, 128, SparseType.INT8), (150, 128, SparseType.INT4), (60, 64, SparseType.FP16),
             (40, 32, SparseType.INT2)]
    mod = IntNBitTableBatchedEmbeddingBagsCodegen(specs)
    tables = [rng.uniform(-1, 1, size=(r, d)).astype(np.float32) for r, d, _ in specs]
    for t, tab in enumerate(tables):
        mod.assign_table(t, torch.from_numpy(tab))
    B = 48
    _, offsets, indices = helpers.ragged_bags(rng, len(specs), B, [r for r, _, _ in specs], 0, 25, 0.1)
    out = mod(torch.from_numpy(indices).cuda(), torch.from_numpy(offsets).cuda())
    assert out.dtype == torch.float16 and out.shape == (B, 128 + 128 + 64 + 32)
    W = mod.weights_dev.cpu().numpy()
    want = oracle.nbit_forward(W, mod.weights_offsets.cpu().numpy(), mod.weights_tys.cpu().numpy(),
                               mod.D_offsets.cpu().numpy(), 16, B, indices, offsets)
    np.testing.assert_allclose(out.float().cpu().numpy(), want, rtol=1e-3, atol=1e-3)
    # and the quantised tables are what the oracle's quantiser makes of the same floats
    for t, (r, d, ty) in enumerate(specs):
        if ty in (SparseType.INT8, SparseType.INT4, SparseType.INT2):
            start, stride = int(mod.weights_offsets[t]), mod.row_strides[t]
            got = W[start:start + r * stride].reshape(r, stride)
            assert np.array_equal(got, oracle.quantize_rows(tables[t], int(ty), 16))
