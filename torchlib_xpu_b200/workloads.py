"""Seeded synthetic inputs for the TBE and jagged configurations.

Host-side numpy generators with a fixed draw order (lengths -> indices -> anything else), so that a
(config, seed) pair always names the same input. They stand in for production traffic: uniform or
bounded-Zipf row ids, uniform bag lengths. Weights are NOT generated here at full size -- the
benchmark fills tables on the device; tests generate small tables with `uniform_table`.
"""
from __future__ import annotations

import dataclasses

import numpy as np


def rng_for(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def bounded_zipf(rng: np.random.Generator, num_rows: int, alpha: float, size: int) -> np.ndarray:
    """Ranks 0..num_rows-1 with p(k) proportional to (k+1)^-alpha, by inverse CDF."""
    cdf = np.cumsum(np.arange(1, num_rows + 1, dtype=np.float64) ** (-alpha))
    cdf /= cdf[-1]
    u = rng.random(size)
    return np.minimum(np.searchsorted(cdf, u, side="left"), num_rows - 1).astype(np.int64)


@dataclasses.dataclass
class TbeInputs:
    T: int
    B: int
    E: int                   # rows per table (all tables alike in the synthetic configs)
    D: int
    lengths: np.ndarray      # int64 [T*B], table-major
    offsets: np.ndarray      # int64 [T*B+1]
    indices: np.ndarray      # int64 [N]

    @property
    def num_lookups(self) -> int:
        return int(self.indices.size)

    def unique_rows(self) -> int:
        """Distinct (table, row) pairs touched."""
        table_of = np.repeat(np.arange(self.T, dtype=np.int64), self.table_lookups())
        return int(np.unique(table_of * self.E + self.indices).size)

    def table_lookups(self) -> np.ndarray:
        ends = self.offsets[self.B::self.B]
        starts = self.offsets[0:self.T * self.B:self.B]
        return ends - starts


def tbe_inputs(T: int, B: int, E: int, D: int, L_lo: int, L_hi: int, seed: int,
               dist: str = "uniform", alpha: float = 1.05, permute: bool = False) -> TbeInputs:
    """Bag lengths ~ integers{L_lo..L_hi}; row ids uniform over [0, E) or bounded Zipf(alpha),
    optionally mapped through one fixed random permutation per table."""
    rng = rng_for(seed)
    lengths = rng.integers(L_lo, L_hi + 1, size=T * B, dtype=np.int64)
    offsets = np.zeros(T * B + 1, dtype=np.int64)
    np.cumsum(lengths, out=offsets[1:])
    n = int(offsets[-1])
    if dist == "uniform":
        indices = rng.integers(0, E, size=n, dtype=np.int64)
    elif dist == "zipf":
        indices = bounded_zipf(rng, E, alpha, n)
        if permute:
            per_table = offsets[B::B] - offsets[0:T * B:B]
            start = 0
            for t in range(T):
                perm = rng.permutation(E)
                stop = start + int(per_table[t])
                indices[start:stop] = perm[indices[start:stop]]
                start = stop
    else:
        raise ValueError("dist must be 'uniform' or 'zipf'")
    return TbeInputs(T=T, B=B, E=E, D=D, lengths=lengths, offsets=offsets, indices=indices)


def uniform_table(rng: np.random.Generator, rows: int, D: int, lo: float, hi: float,
                  dtype=np.float32) -> np.ndarray:
    return rng.uniform(lo, hi, size=(rows, D)).astype(np.float32).astype(dtype)


@dataclasses.dataclass
class JaggedInputs:
    B: int
    max_L: int
    D: int
    lengths: np.ndarray      # int64 [B]
    offsets: np.ndarray      # int64 [B+1]

    @property
    def total_rows(self) -> int:
        return int(self.offsets[-1])


def jagged_inputs(B: int, max_L: int, D: int, seed: int) -> JaggedInputs:
    rng = rng_for(seed)
    lengths = rng.integers(0, max_L + 1, size=B, dtype=np.int64)
    offsets = np.zeros(B + 1, dtype=np.int64)
    np.cumsum(lengths, out=offsets[1:])
    return JaggedInputs(B=B, max_L=max_L, D=D, lengths=lengths, offsets=offsets)


# The five named configurations (sizes only; see tbe_inputs / jagged_inputs for the draws).
CONFIGS = {
    "tbe_fp32_fwd": dict(T=8, E=100_000, D=128, B=2048, L_lo=1, L_hi=40, dist="uniform", seed=0),
    "jagged": dict(B=4096, max_L=128, D=256, seed=1),
    "tbe_fp16_train": dict(T=26, E=1_000_000, D=128, B=8192, L_lo=1, L_hi=64, dist="zipf",
                           alpha=1.05, permute=True, seed=2),
    "tbe_nbit_fwd": dict(T=64, E=2_000_000, D=128, B=16384, L_lo=1, L_hi=100, dist="zipf",
                         alpha=1.1, permute=False, seed=3),
    "tbe_sharded": dict(T_per_gpu=64, E=4_000_000, D=128, B=65536, L_lo=1, L_hi=50, dist="zipf",
                        alpha=1.05, permute=False, seed=4),
}


def forward_bytes(N: int, U: int, row_bytes: int, T: int, B: int, D: int, out_elem: int) -> int:
    """Compulsory bytes of a pooled forward: distinct rows once + indices + offsets + output."""
    return U * row_bytes + N * 8 + (T * B + 1) * 8 + B * T * D * out_elem


def backward_bytes(N: int, U: int, row_bytes: int, T: int, B: int, D: int, grad_elem: int) -> int:
    """Compulsory bytes of backward + row-wise Adagrad: gradient once, indices, offsets, and a
    read + write of every distinct row with its 4-byte state."""
    return B * T * D * grad_elem + N * 8 + (T * B + 1) * 8 + U * (2 * row_bytes + 8)
