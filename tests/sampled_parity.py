"""Parity checks on full-size problems by sampling.

At the sizes of the named configurations the CPU oracle cannot pool every bag or update every row
in reasonable time, and the tables (tens of GB) are generated on the device. What a pooled vector
or an updated row depends on is small, though: a bag needs only the rows it names, a row's update
only the lookups that name it. So a check draws a sample of bags (or rows), reads exactly what they
depend on back from the device, builds a compact problem out of it -- the sampled rows renumbered
into a small table -- runs the ORACLE on that, and compares with what the CUDA kernels produced for
the same bags (rows) in the full-size run. The comparison is against the oracle's arithmetic, with
device memory used only as the place the inputs happen to live.

Everything takes torch tensors (ids and offsets may live on the device or the host).
"""
from __future__ import annotations

import numpy as np
import torch

import oracle


def _np(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def _bag_positions(offsets: torch.Tensor, first_bag: int, bags: torch.Tensor):
    """Lookup positions of the sampled bags of one table, and the compact offsets array."""
    starts = offsets[first_bag + bags].to(torch.int64)
    ends = offsets[first_bag + bags + 1].to(torch.int64)
    lens = ends - starts
    compact = torch.zeros(bags.numel() + 1, dtype=torch.int64, device=offsets.device)
    torch.cumsum(lens, 0, out=compact[1:])
    total = int(compact[-1].item())
    # position k of the compact array belongs to bag j = searchsorted(compact, k, right) - 1
    k = torch.arange(total, device=offsets.device)
    j = torch.searchsorted(compact, k, right=True) - 1
    return starts[j] + (k - compact[j]), compact


def forward_sample_check(dev_weights, row_elems_or_bytes, table_base, D_begin, D, weights_ty, indices,
                         offsets, B, t, pooled, bags, rtol, atol, pooling_mode=oracle.SUM,
                         per_sample_weights=None, row_alignment=16, pooled_row0=0):
    """Checks the pooled vectors of `bags` (1-D int64 tensor of sample numbers) of table t.

    dev_weights: the flat table buffer on the device; table_base: element (float tables) or byte
    (quantised tables) offset of the table's row 0; row_elems_or_bytes: elements per row of a float
    table, bytes per row of a quantised one. weights_ty: oracle.FP32 / FP16 / INT8 / INT4 / INT2.
    pooled: the [*, total_D] result of the CUDA forward; pooled_row0: sample number of its row 0.
    Returns the number of bags compared."""
    dev = dev_weights.device
    bags = bags.to(offsets.device)
    pos, compact = _bag_positions(offsets, t * B, bags)
    ids = indices[pos].to(torch.int64)
    uniq, inv = torch.unique(ids, return_inverse=True)
    stride = int(row_elems_or_bytes)
    cols = torch.arange(stride, device=dev)
    rows = dev_weights.view(-1)[(table_base + uniq.to(dev)[:, None] * stride + cols[None, :])]
    psw = None if per_sample_weights is None else _np(per_sample_weights[pos])
    n = bags.numel()
    quantised = weights_ty in (oracle.INT8, oracle.INT4, oracle.INT2)
    if quantised:
        want = oracle.nbit_forward(_np(rows).reshape(-1), np.zeros(1, np.int64), np.array([weights_ty], np.uint8),
                                   np.array([0, D], np.int32), row_alignment, n, _np(inv), _np(compact), psw,
                                   pooling_mode)
    else:
        want = oracle.tbe_forward(_np(rows).reshape(-1), weights_ty, np.zeros(1, np.int64),
                                  np.array([0, D], np.int32), n, _np(inv), _np(compact), psw, pooling_mode)
    got = _np(pooled[(bags.to(pooled.device) - pooled_row0), D_begin:D_begin + D].float())
    np.testing.assert_allclose(got, want, rtol=rtol, atol=atol,
                               err_msg="pooled vectors of table %d differ from the oracle" % t)
    return n


class BackwardSample:
    """Rows of one table whose update is checked: the `hot` most looked-up rows plus `extra` random
    ones among those the batch touches. Construct BEFORE the CUDA backward (it reads the rows and
    their optimizer state as they are), call check() after it."""

    def __init__(self, dev_weights, table_base, D, weights_ty, momentum, momentum_base, indices, offsets,
                 B, t, hot=64, extra=1000, seed=0):
        self.t, self.D, self.B, self.ty = t, D, B, weights_ty
        self.table_base, self.momentum_base = table_base, momentum_base
        a, b = int(offsets[t * B].item()), int(offsets[(t + 1) * B].item())
        ids = indices[a:b].to(torch.int64)
        uniq, counts = torch.unique(ids, return_counts=True)
        order = torch.argsort(counts, descending=True)
        pick = [uniq[order[:hot]]]
        if uniq.numel() > hot and extra > 0:
            g = torch.Generator(device="cpu").manual_seed(seed)
            rest = order[hot:]
            take = rest[torch.randperm(rest.numel(), generator=g)[:extra].to(rest.device)]
            pick.append(uniq[take])
        self.rows = torch.sort(torch.cat(pick)).values                    # sampled row ids, ascending
        self.max_run = int(counts.max().item()) if counts.numel() else 0
        # the lookups that name a sampled row, as a compact problem over the same B bags
        hit = torch.isin(ids, self.rows)
        pos = torch.nonzero(hit).flatten()                                # relative to a
        self.pos = pos + a
        bag_of = torch.searchsorted(offsets[t * B:(t + 1) * B + 1].to(torch.int64), self.pos, right=True) - 1
        per_bag = torch.bincount(bag_of, minlength=B)
        self.offsets = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(_np(per_bag), out=self.offsets[1:])
        self.ids = _np(torch.searchsorted(self.rows, ids[pos]))           # renumbered
        dev = dev_weights.device
        cols = torch.arange(D, device=dev)
        self._gather = (table_base + self.rows.to(dev)[:, None] * D + cols[None, :])
        self.w_old = _np(dev_weights.view(-1)[self._gather]).copy()
        self.m_old = None
        if momentum is not None:
            self.m_old = _np(momentum[momentum_base + self.rows.to(momentum.device)]).copy()

    def check(self, dev_weights, momentum, grad, D_begin, optimizer, lr, eps, rtol=1e-3, atol=1e-3,
              update_rtol=1e-2, per_sample_weights=None, pooling_mode=oracle.SUM):
        """grad: the [B, total_D] gradient matrix the CUDA backward read (device or host)."""
        D, B = self.D, self.B
        g = _np(grad[:, D_begin:D_begin + D].float())
        w_ref = self.w_old.reshape(-1).copy()
        m_ref = None if self.m_old is None else self.m_old.copy()
        psw = None if per_sample_weights is None else _np(per_sample_weights[self.pos])
        nrows = self.rows.numel()
        oracle.tbe_backward(w_ref, self.ty, np.zeros(1, np.int64), np.array([0, D], np.int32),
                            np.array([0, nrows], np.int64), B, self.ids, self.offsets, g, m_ref,
                            None if m_ref is None else np.zeros(1, np.int64), optimizer, lr, eps, psw,
                            pooling_mode)
        got = _np(dev_weights.view(-1)[self._gather]).astype(np.float32)
        want = w_ref.reshape(nrows, D).astype(np.float32)
        np.testing.assert_allclose(got, want, rtol=rtol, atol=atol,
                                   err_msg="updated rows of table %d differ from the oracle" % self.t)
        old = self.w_old.astype(np.float32)
        moved = np.abs(want - old).max(axis=1) > 0
        assert moved.any(), "the sample holds no row that the oracle moves"
        # the updates themselves, not just the small weights they were applied to (an fp16 weight
        # moves in steps of its spacing: two spacings of slack)
        slack = 2 * float(np.spacing(np.float16(np.abs(want).max()))) if self.ty == oracle.FP16 else 1e-7
        np.testing.assert_allclose(got - old, want - old, rtol=update_rtol, atol=slack,
                                   err_msg="updates of table %d differ from the oracle" % self.t)
        if m_ref is not None:
            got_m = _np(momentum[self.momentum_base + self.rows.to(momentum.device)])
            np.testing.assert_allclose(got_m, m_ref, rtol=1e-4, atol=1e-6,
                                       err_msg="optimizer state of table %d differs" % self.t)
        return nrows
