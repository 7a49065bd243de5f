"""GPU parity over seeded random shapes: table counts, batch sizes on both sides of the point where a
warp takes a group of bags, row widths of every lane grouping, bag lengths, empty bags, pooling modes,
per-sample weights, id widths, ids out of range, several destination buffers -- each case against the
CPU oracle with the tolerances of the fixed-shape tests."""
import numpy as np
import pytest
import torch

import oracle
from tests import helpers
from tests.test_backward_gpu import _backward_case, _check
from torchlib_xpu_b200 import cabi

pytestmark = pytest.mark.gpu

BATCHES = [1, 7, 33, 500, 12000, 24001, 47361, 60000]


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _bags_with_bad_ids(rng, T, B, rows, weighted):
    L_hi = int(rng.choice([1, 3, 12, 40]))
    L_lo = int(rng.integers(0, L_hi + 1))
    _, offsets, indices = helpers.ragged_bags(rng, T, B, rows, L_lo, L_hi,
                                              empty_fraction=float(rng.choice([0, 0.3, 0.9])))
    psw = rng.random(indices.size).astype(np.float32) if weighted else None
    n_bad = int(min(indices.size, rng.choice([0, 0, 5])))
    keep = np.ones(indices.size, dtype=np.float32)
    bad = indices.copy()
    if n_bad:
        at = rng.choice(indices.size, size=n_bad, replace=False)
        bad[at] = 100000
        keep[at] = 0
    # flagged lookups contribute nothing: the oracle sees them with weight zero
    oracle_w = (keep if psw is None else psw * keep) if (n_bad or psw is not None) else None
    return offsets, indices, bad, keep, psw, oracle_w, n_bad


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_forward_random_shapes(seed):
    rng = np.random.default_rng(seed)
    for _ in range(12):
        T, B = int(rng.integers(1, 5)), int(rng.choice(BATCHES))
        wd = rng.choice([np.float32, np.float16])
        widths = [4, 8, 20, 32, 64, 72, 100, 128] + ([256] if wd == np.float16 else [])
        Ds = [int(rng.choice(widths)) for _ in range(T)]
        rows = [int(rng.integers(1, 3000)) for _ in range(T)]
        weighted, pooling = bool(rng.integers(0, 2)), int(rng.choice([oracle.SUM, oracle.MEAN]))
        idt = rng.choice([np.int32, np.int64])
        W, wo, Do = helpers.float_tables(rng, rows, Ds, wd, -1.0, 1.0)
        offsets, indices, bad, keep, psw, oracle_w, n_bad = _bags_with_bad_ids(rng, T, B, rows, weighted)
        want = oracle.tbe_forward(W, oracle.FP32 if wd == np.float32 else oracle.FP16, wo, Do, B,
                                  np.where(keep > 0, indices, 0), offsets, oracle_w, pooling)
        G = int(rng.choice([1, 1, 2, 3]))
        rpd, total_D = (B + G - 1) // G, int(Do[-1])
        odt = torch.float32 if rng.integers(0, 2) else torch.float16
        bufs = [torch.full((rpd, total_D + 8), -7.0, dtype=odt, device="cuda") for _ in range(G)]
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        cabi.forward(_dev(W), _dev(wo), _dev(Do), total_D, max(Ds), _dev(bad.astype(idt)), _dev(offsets.astype(idt)),
                     B, pooling, None if psw is None else _dev(psw), odt, _dev(np.asarray(rows, dtype=np.int64)),
                     status, outputs=bufs, output_stride=total_D + 8, output_col_offset=4, rows_per_dest=rpd)
        torch.cuda.synchronize()
        got = torch.cat([b[:, 4:4 + total_D] for b in bufs])[:B].float().cpu().numpy()
        what = dict(T=T, B=B, Ds=Ds, weights=wd.__name__, pooling=pooling, weighted=weighted, dests=G)
        for b in bufs:
            assert bool((b[:, :4] == -7).all()) and bool((b[:, 4 + total_D:] == -7).all()), what
        assert bool(status.item() & cabi.DEV_INDEX_OUT_OF_RANGE) == bool(n_bad), what
        tol = dict(rtol=1e-5, atol=2e-5) if (wd == np.float32 and odt == torch.float32) else dict(rtol=2e-3, atol=2e-3)
        np.testing.assert_allclose(got, want, err_msg=str(what), **tol)


@pytest.mark.parametrize("seed", [21, 22, 23])
def test_nbit_forward_random_shapes(seed):
    rng = np.random.default_rng(seed)
    for _ in range(12):
        T, B = int(rng.integers(1, 5)), int(rng.choice(BATCHES))
        tys = [int(rng.choice([oracle.INT8, oracle.INT4, oracle.INT8, oracle.INT4, oracle.INT2, oracle.FP16]))
               for _ in range(T)]
        Ds = [int(rng.choice([4, 8, 20, 64, 68, 128, 256] if ty == oracle.INT8 else [8, 16, 40, 64, 128, 256]))
              for ty in tys]
        rows = [int(rng.integers(1, 3000)) for _ in range(T)]
        align = int(rng.choice([16, 16, 1, 4]))
        weighted, pooling = bool(rng.integers(0, 2)), int(rng.choice([oracle.SUM, oracle.MEAN]))
        idt = rng.choice([np.int32, np.int64])
        W, wo, Do, tys_a = helpers.quantised_tables(rng, rows, Ds, tys, align)
        offsets, indices, bad, keep, psw, oracle_w, n_bad = _bags_with_bad_ids(rng, T, B, rows, weighted)
        want = oracle.nbit_forward(W, wo, tys_a, Do, align, B, np.where(keep > 0, indices, 0), offsets, oracle_w,
                                   pooling)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        got = cabi.nbit_forward(_dev(W), _dev(wo), _dev(tys_a), _dev(Do), int(Do[-1]), max(Ds),
                                _dev(bad.astype(idt)), _dev(offsets.astype(idt)), B, pooling,
                                None if psw is None else _dev(psw), torch.float32, align,
                                _dev(np.asarray(rows, dtype=np.int64)), status,
                                table_types=set(int(t) for t in tys) if rng.integers(0, 2) else None)
        torch.cuda.synchronize()
        what = dict(T=T, B=B, tys=tys, Ds=Ds, align=align, pooling=pooling, weighted=weighted)
        assert bool(status.item() & cabi.DEV_INDEX_OUT_OF_RANGE) == bool(n_bad), what
        np.testing.assert_allclose(got.cpu().numpy(), want, rtol=2e-3, atol=2e-3, err_msg=str(what))


@pytest.mark.parametrize("seed", [31, 32])
def test_backward_random_shapes(seed):
    rng = np.random.default_rng(seed)
    for _ in range(12):
        T, B = int(rng.integers(1, 5)), int(rng.choice([1, 9, 100, 2000, 9000]))
        wd, gd = rng.choice([np.float32, np.float16]), rng.choice([np.float32, np.float16])
        max_D = int(rng.choice([32, 64, 128, 256, 512]))
        Ds = [int(rng.choice([d for d in (8, 16, 32, 64, 128, 256, 512) if d <= max_D])) for _ in range(T)]
        rows = [int(rng.integers(1, 5000)) for _ in range(T)]
        L_hi = int(rng.choice([1, 4, 20, 60]))
        L_lo = int(rng.integers(0, L_hi + 1))
        pooling = int(rng.choice([oracle.SUM, oracle.MEAN]))
        opt = int(rng.choice([oracle.ROWWISE_ADAGRAD, oracle.SGD]))
        weighted = bool(rng.integers(0, 2))
        hot = int(rng.integers(0, rows[0])) if rng.integers(0, 2) else None     # a run of most of table 0's lookups
        case = _backward_case(rng, rows, Ds, B, L_lo, L_hi, wd, gd, pooling, opt, weighted, hot_row=hot)
        _check(*case, B, wd, gd, pooling, opt, idx_dtype=rng.choice([np.int32, np.int64]), lr=0.01,
               rows_hint=bool(rng.integers(0, 2)))
