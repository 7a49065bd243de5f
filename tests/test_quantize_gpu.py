"""GPU parity: row-wise quantise / dequantise kernels vs the CPU oracle and FBGEMM-core."""
import numpy as np
import pytest
import torch

import oracle
import torchlib_xpu_b200
from torchlib_xpu_b200 import cabi, workloads

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("ty,D", [(oracle.INT8, 128), (oracle.INT4, 128), (oracle.INT2, 64),
                                  (oracle.INT8, 20), (oracle.INT4, 36), (oracle.INT4, 1024)])
@pytest.mark.parametrize("row_alignment", [16, 1])
def test_quantize_rows_matches_oracle_bit_for_bit(ty, D, row_alignment):
    rng = workloads.rng_for(600 + D)
    src = rng.uniform(-1, 1, size=(513, D)).astype(np.float32)
    src[7] = 0.125       # zero range
    src[8, :] = 0.0
    want = oracle.quantize_rows(src, ty, row_alignment)
    got = cabi.quantize_rows(torch.from_numpy(src).cuda(), ty, row_alignment).cpu().numpy()
    assert got.shape == want.shape
    assert np.array_equal(got, want)          # integer/byte work: exact
    back = cabi.dequantize_rows(torch.from_numpy(want).cuda(), D, ty, row_alignment).cpu().numpy()
    stride1 = oracle.nbit_row_stride(ty, D, 1)
    ref = oracle.dequantize_rows_ref(np.ascontiguousarray(want[:, :stride1]), D, ty)
    np.testing.assert_allclose(back, ref, rtol=1e-6, atol=1e-7)


def test_quantize_fp16_source_and_table_roundtrip_through_lookup():
    """Tables quantised on the GPU feed the quantised lookup and agree with the oracle."""
    rng = workloads.rng_for(601)
    D, E, B = 128, 300, 32
    src = rng.uniform(-1, 1, size=(E, D)).astype(np.float16)
    rows_gpu = cabi.quantize_rows(torch.from_numpy(src).cuda(), oracle.INT4, 16)
    want_rows = oracle.quantize_rows(src.astype(np.float32), oracle.INT4, 16)
    assert np.array_equal(rows_gpu.cpu().numpy(), want_rows)
    lengths = rng.integers(0, 20, size=B)
    offsets = np.zeros(B + 1, dtype=np.int64)
    np.cumsum(lengths, out=offsets[1:])
    indices = rng.integers(0, E, size=offsets[-1])
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    out = cabi.nbit_forward(rows_gpu.reshape(-1), dev(np.zeros(1, np.int64)),
                            dev(np.array([oracle.INT4], np.uint8)), dev(np.array([0, D], np.int32)), D, D,
                            dev(indices), dev(offsets), B, output_dtype=torch.float32)
    want = oracle.nbit_forward(want_rows.reshape(-1), [0], [oracle.INT4], [0, D], 16, B, indices, offsets)
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=1e-3, atol=1e-3)


def test_fused_nbit_ops_use_the_fbgemm_op_layout():
    torchlib_xpu_b200.load_torch_ops()
    rng = workloads.rng_for(602)
    src = rng.uniform(-2, 2, size=(100, 64)).astype(np.float32)
    for bit_rate, ty in ((8, oracle.INT8), (4, oracle.INT4), (2, oracle.INT2)):
        q = torch.ops.fbgemm.FloatToFusedNBitRowwiseQuantizedSBHalf(torch.from_numpy(src).cuda(), bit_rate)
        ref = oracle.quantize_rows(src, ty, 1, backend="ref")    # FBGEMM-core, header first
        payload = ref.shape[1] - 4
        tail = np.concatenate([ref[:, 4:], ref[:, :4]], axis=1)   # FBGEMM op layout: header last
        got = q.cpu().numpy()
        assert got.shape == tail.shape
        assert np.array_equal(got[:, payload:], tail[:, payload:])        # scale / bias exact
        assert np.mean(got == tail) > 0.995                                # ties may differ by one step
        back = torch.ops.fbgemm.FusedNBitRowwiseQuantizedSBHalfToFloat(q, bit_rate).cpu().numpy()
        scale = ref[:, :2].copy().view(np.float16).astype(np.float32)
        assert np.all(np.abs(back - src) <= scale * 0.51 + 2e-3)
        half = torch.ops.fbgemm.FusedNBitRowwiseQuantizedSBHalfToFloatOrHalf(q, bit_rate, 1)
        assert half.dtype == torch.float16
