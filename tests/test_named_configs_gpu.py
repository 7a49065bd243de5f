"""The named training and quantised-inference configurations at their full size, and a table beyond
64 GB, checked against the oracle by sampling (tests/sampled_parity.py): the regimes small cases do
not reach -- 25-bit key spaces, runs of tens of thousands of lookups next to millions of single
ones, row offsets that need more than 36 bits."""
import numpy as np
import pytest
import torch

import oracle
from tests import sampled_parity
from torchlib_xpu_b200 import cabi, workloads

pytestmark = pytest.mark.gpu


def _half_table(num_elems, lo, hi, gen):
    w = torch.empty(num_elems, dtype=torch.float16, device="cuda")
    chunk = 1 << 28
    for a in range(0, num_elems, chunk):
        b = min(num_elems, a + chunk)
        w[a:b] = (torch.rand(b - a, device="cuda", generator=gen) * (hi - lo) + lo).half()
    return w


def _sample_bags(B, count, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.sort(torch.randperm(B, generator=g)[:count]).values


def test_training_config_full_size_forward_and_backward():
    """T=26 fp16 tables x 1 M rows x D=128, B=8192, L~U{1..64}, Zipf(1.05) ids through a fixed
    permutation, fp32 gradients, row-wise Adagrad lr 0.01 eps 1e-8 (6.9 M lookups, 1.7 M distinct
    rows, hottest row ~25 k lookups). Forward: 256 bags of every table. Backward: the 64 hottest
    rows and 1000 random touched rows of every table."""
    c = workloads.CONFIGS["tbe_fp16_train"]
    T, E, D, B = c["T"], c["E"], c["D"], c["B"]
    inp = workloads.tbe_inputs(T, B, E, D, c["L_lo"], c["L_hi"], c["seed"], "zipf", c["alpha"], c["permute"])
    gen = torch.Generator(device="cuda").manual_seed(1234)
    W = _half_table(T * E * D, -0.01, 0.01, gen)
    mom = torch.rand(T * E, device="cuda", generator=gen) * 0.05
    wo = torch.arange(T, device="cuda", dtype=torch.int64) * (E * D)
    Do = torch.arange(T + 1, device="cuda", dtype=torch.int32) * D
    hs = torch.arange(T + 1, device="cuda", dtype=torch.int64) * E
    idx, offs = torch.from_numpy(inp.indices).cuda(), torch.from_numpy(inp.offsets).cuda()
    grad = torch.randn((B, T * D), device="cuda", generator=gen)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rows = torch.full((T,), E, dtype=torch.int64, device="cuda")

    out = cabi.forward(W, wo, Do, T * D, D, idx, offs, B, rows_per_table=rows, status=status)
    checked = 0
    for t in range(T):
        checked += sampled_parity.forward_sample_check(W, D, t * E * D, t * D, D, oracle.FP16, idx, offs, B, t,
                                                       out, _sample_bags(B, 256, 100 + t), 1e-3, 1e-3)
    assert checked == 256 * T

    samples = [sampled_parity.BackwardSample(W, t * E * D, D, oracle.FP16, mom, t * E, idx, offs, B, t,
                                             hot=64, extra=1000, seed=t) for t in range(T)]
    assert max(s.max_run for s in samples) > 10_000      # the regime this test is for
    bits = (T * E - 1).bit_length()
    cabi.backward(W, wo, Do, hs, bits, D, idx, offs, B, grad, cabi.OPT_ROWWISE_ADAGRAD, 0.01, 1e-8, mom,
                  hs[:-1].clone(), status=status, max_table_rows=E)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for t, s in enumerate(samples):
        s.check(W, mom, grad, t * D, oracle.ROWWISE_ADAGRAD, 0.01, 1e-8)


def test_quantised_inference_config_full_size():
    """T=64 tables x 2 M rows x D=128, the first half INT8 and the second INT4 with fp16 scale/bias
    leading every row (14.3 GB), B=16384, L~U{1..100}, Zipf(1.1) ids, fp16 output: 256 bags of every
    table against the oracle's dequantise-and-pool."""
    c = workloads.CONFIGS["tbe_nbit_fwd"]
    T, E, D, B = c["T"], c["E"], c["D"], c["B"]
    inp = workloads.tbe_inputs(T, B, E, D, c["L_lo"], c["L_hi"], c["seed"], "zipf", c["alpha"])
    gen = torch.Generator(device="cuda").manual_seed(4321)
    tys = [oracle.INT8 if t < T // 2 else oracle.INT4 for t in range(T)]
    strides = [oracle.nbit_row_stride(ty, D, 16) for ty in tys]
    wo_host = np.zeros(T, dtype=np.int64)
    np.cumsum([E * s for s in strides[:-1]], out=wo_host[1:])
    Wq = torch.empty(int(wo_host[-1]) + E * strides[-1], dtype=torch.uint8, device="cuda")
    # every table is a real quantisation of U(-1, 1) rows, made by the library's own quantiser in
    # slices (b200tbe_quantize_rows is checked bit for bit against the oracle elsewhere)
    slice_rows = 250_000
    for t in range(T):
        tab = Wq[int(wo_host[t]):int(wo_host[t]) + E * strides[t]].view(E, strides[t])
        for a in range(0, E, slice_rows):
            src = torch.rand((min(slice_rows, E - a), D), device="cuda", generator=gen) * 2 - 1
            tab[a:a + src.shape[0]] = cabi.quantize_rows(src, tys[t], 16, header_first=True)
    wo = torch.from_numpy(wo_host).cuda()
    Do = torch.arange(T + 1, device="cuda", dtype=torch.int32) * D
    tys_dev = torch.tensor(tys, dtype=torch.uint8, device="cuda")
    idx, offs = torch.from_numpy(inp.indices).cuda(), torch.from_numpy(inp.offsets).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rows = torch.full((T,), E, dtype=torch.int64, device="cuda")
    out = cabi.nbit_forward(Wq, wo, tys_dev, Do, T * D, D, idx, offs, B, rows_per_table=rows, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and out.dtype == torch.float16
    for t in range(T):
        # fp16 output: half an fp16 spacing of the pooled value on top of the north-star tolerance
        sampled_parity.forward_sample_check(Wq, strides[t], int(wo_host[t]), t * D, D, tys[t], idx, offs, B, t,
                                            out, _sample_bags(B, 256, 300 + t), 2e-3, 1e-3)


def test_forward_of_a_table_beyond_64_gb():
    """One fp32 table of 68 M rows x D=256 (69.6 GB; rows of 1 KB run on the ring engine): ids in the
    last part of the table have byte offsets beyond 2^36. The table is not initialised as a whole;
    the rows the bags name are."""
    free, _ = torch.cuda.mem_get_info()
    E, D, B, L = 68_000_000, 256, 512, 24
    if free < E * D * 4 + (4 << 30):
        pytest.skip("needs 74 GB of free device memory")
    W = torch.empty(E * D, dtype=torch.float32, device="cuda")
    rng = workloads.rng_for(77)
    first_far = (1 << 36) // (D * 4) + 1
    ids = rng.integers(first_far, E, size=B * L, dtype=np.int64)
    ids[::7] = rng.integers(0, 1000, size=ids[::7].size)           # near rows in the same bags
    ids[5] = E - 1
    uniq = np.unique(ids)
    vals = rng.uniform(-1, 1, size=(uniq.size, D)).astype(np.float32)
    W.view(E, D)[torch.from_numpy(uniq).cuda()] = torch.from_numpy(vals).cuda()
    offsets = np.arange(B + 1, dtype=np.int64) * L
    wo = torch.zeros(1, dtype=torch.int64, device="cuda")
    Do = torch.tensor([0, D], dtype=torch.int32, device="cuda")
    idx, offs = torch.from_numpy(ids).cuda(), torch.from_numpy(offsets).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = cabi.forward(W, wo, Do, D, D, idx, offs, B, rows_per_table=torch.tensor([E], device="cuda"),
                       status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    n = sampled_parity.forward_sample_check(W, D, 0, 0, D, oracle.FP32, idx, offs, B, 0, out,
                                            torch.arange(B), 1e-5, 1e-6)
    assert n == B
    del W
    torch.cuda.empty_cache()
