"""Small shared builders for the tests: table layouts in the TBE conventions, as numpy."""
from __future__ import annotations

import numpy as np

import oracle
from torchlib_xpu_b200 import workloads


def float_tables(rng, rows_per_table, Ds, dtype, lo=-0.01, hi=0.01):
    """Flat dev_weights + weights_offsets (elements) + D_offsets for fp32/fp16 tables."""
    tables = [workloads.uniform_table(rng, r, d, lo, hi, dtype) for r, d in zip(rows_per_table, Ds)]
    weights_offsets = np.zeros(len(Ds), dtype=np.int64)
    pos = 0
    for t, tab in enumerate(tables):
        weights_offsets[t] = pos
        pos += tab.size
    dev_weights = np.concatenate([tab.reshape(-1) for tab in tables]) if tables else np.zeros(0, dtype)
    D_offsets = np.zeros(len(Ds) + 1, dtype=np.int32)
    np.cumsum(np.asarray(Ds, dtype=np.int32), out=D_offsets[1:])
    return dev_weights, weights_offsets, D_offsets


def quantised_tables(rng, rows_per_table, Ds, tys, row_alignment, backend="c"):
    """Byte buffer of mixed INT8/INT4/INT2/FP16/FP32 tables in the quantised-op layout."""
    chunks, weights_offsets, pos = [], np.zeros(len(Ds), dtype=np.int64), 0
    for t, (r, d, ty) in enumerate(zip(rows_per_table, Ds, tys)):
        src = rng.uniform(-1.0, 1.0, size=(r, d)).astype(np.float32)
        if ty in (oracle.INT8, oracle.INT4, oracle.INT2):
            rows = oracle.quantize_rows(src, ty, row_alignment, backend=backend)
        else:
            elem = np.float16 if ty == oracle.FP16 else np.float32
            stride = oracle.nbit_row_stride(ty, d, row_alignment)
            rows = np.zeros((r, stride), dtype=np.uint8)
            raw = src.astype(elem).view(np.uint8).reshape(r, -1)
            rows[:, :raw.shape[1]] = raw
        # every table starts on a 16-byte boundary, as GPU tables do
        pad = (-pos) % 16
        if pad:
            chunks.append(np.zeros(pad, dtype=np.uint8))
            pos += pad
        weights_offsets[t] = pos
        chunks.append(rows.reshape(-1))
        pos += rows.size
    dev_weights = np.concatenate(chunks) if chunks else np.zeros(0, np.uint8)
    D_offsets = np.zeros(len(Ds) + 1, dtype=np.int32)
    np.cumsum(np.asarray(Ds, dtype=np.int32), out=D_offsets[1:])
    return dev_weights, weights_offsets, D_offsets, np.asarray(tys, dtype=np.uint8)


def ragged_bags(rng, T, B, rows_per_table, L_lo, L_hi, empty_fraction=0.0):
    """Table-major bags with per-table row ranges; some bags forced empty."""
    lengths = rng.integers(L_lo, L_hi + 1, size=T * B, dtype=np.int64)
    if empty_fraction > 0:
        lengths[rng.random(T * B) < empty_fraction] = 0
    offsets = np.zeros(T * B + 1, dtype=np.int64)
    np.cumsum(lengths, out=offsets[1:])
    indices = np.zeros(int(offsets[-1]), dtype=np.int64)
    for t in range(T):
        a, b = int(offsets[t * B]), int(offsets[(t + 1) * B])
        indices[a:b] = rng.integers(0, rows_per_table[t], size=b - a, dtype=np.int64)
    return lengths, offsets, indices
