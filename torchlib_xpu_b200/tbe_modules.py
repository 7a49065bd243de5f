"""Module facades over the fbgemm operators, in the shape of fbgemm_gpu's
SplitTableBatchedEmbeddingBagsCodegen (training) and IntNBitTableBatchedEmbeddingBagsCodegen
(quantised inference): they own the flat weight buffer, the per-table offset tables and the
optimizer state, and call torch.ops.fbgemm.* -- nothing is computed in Python.

Only what the CUDA kernels implement is accepted: all tables in device memory, exact SGD or exact
row-wise Adagrad, SUM / MEAN pooling, fp32 / fp16 training weights, INT8 / INT4 / INT2 / FP16 / FP32
inference tables.
"""
from __future__ import annotations

import enum
from typing import List, Optional, Sequence, Tuple

import torch

from . import cabi, load_torch_ops


class PoolingMode(enum.IntEnum):
    SUM = 0
    MEAN = 1


class SparseType(enum.IntEnum):
    FP32 = 0
    FP16 = 1
    INT8 = 2
    INT4 = 3
    INT2 = 4


class OptimType(enum.Enum):
    EXACT_SGD = "exact_sgd"
    EXACT_ROWWISE_ADAGRAD = "exact_row_wise_adagrad"


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


class SplitTableBatchedEmbeddingBagsCodegen(torch.nn.Module):
    """Training tables: embedding_specs is [(rows, dim), ...]; the backward pass applies the
    optimizer in place (no weight gradient is produced)."""

    def __init__(self, embedding_specs: Sequence[Tuple[int, int]],
                 optimizer: OptimType = OptimType.EXACT_ROWWISE_ADAGRAD, learning_rate: float = 0.01,
                 eps: float = 1e-8, pooling_mode: PoolingMode = PoolingMode.SUM,
                 weights_precision: SparseType = SparseType.FP32,
                 output_dtype: SparseType = SparseType.FP32, device="cuda",
                 weights_dev: Optional[torch.Tensor] = None,
                 momentum1_dev: Optional[torch.Tensor] = None):
        """weights_dev / momentum1_dev: adopt existing flat buffers (tables too large to hold twice)
        instead of allocating and initialising new ones; they are updated in place."""
        super().__init__()
        load_torch_ops()
        if weights_precision not in (SparseType.FP32, SparseType.FP16):
            raise ValueError("training weights are FP32 or FP16")
        for rows, dim in embedding_specs:
            if dim % 4 != 0 or rows <= 0:
                raise ValueError("every table needs rows > 0 and a dim that is a multiple of 4")
        self.embedding_specs = [(int(r), int(d)) for r, d in embedding_specs]
        self.optimizer, self.learning_rate, self.eps = optimizer, float(learning_rate), float(eps)
        self.pooling_mode, self.output_dtype = PoolingMode(pooling_mode), SparseType(output_dtype)
        dev = torch.device(device)
        wdtype = torch.float32 if weights_precision == SparseType.FP32 else torch.float16
        T = len(self.embedding_specs)
        w_off, h_cum, d_off, pos, rows_total = [], [0], [0], 0, 0
        for rows, dim in self.embedding_specs:
            w_off.append(pos)
            pos += rows * dim
            rows_total += rows
            h_cum.append(rows_total)
            d_off.append(d_off[-1] + dim)
        self.total_D, self.max_D = d_off[-1], max(d for _, d in self.embedding_specs)
        self.total_hash_size_bits = max(1, (rows_total - 1).bit_length())
        if weights_dev is not None and (weights_dev.numel() != pos or weights_dev.dtype != wdtype):
            raise ValueError("weights_dev must hold %d %s elements" % (pos, wdtype))
        self.weights_dev = torch.nn.Parameter(
            weights_dev if weights_dev is not None else torch.empty(pos, dtype=wdtype, device=dev),
            requires_grad=False)
        self.register_buffer("weights_offsets", torch.tensor(w_off, dtype=torch.int64, device=dev))
        self.register_buffer("D_offsets", torch.tensor(d_off, dtype=torch.int32, device=dev))
        self.register_buffer("hash_size_cumsum", torch.tensor(h_cum, dtype=torch.int64, device=dev))
        if momentum1_dev is not None and (momentum1_dev.numel() != rows_total or momentum1_dev.dtype != torch.float32):
            raise ValueError("momentum1_dev must hold %d float32 elements" % rows_total)
        self.register_buffer("momentum1_dev", momentum1_dev if momentum1_dev is not None else torch.zeros(
            rows_total if optimizer == OptimType.EXACT_ROWWISE_ADAGRAD else 0, dtype=torch.float32, device=dev))
        self.register_buffer("momentum1_offsets", torch.tensor(h_cum[:-1], dtype=torch.int64, device=dev))
        self.register_buffer("_placeholder", torch.zeros(1, device=dev))
        self._empty_w = torch.empty(0, dtype=wdtype, device=dev)
        self._empty_f = torch.empty(0, dtype=torch.float32, device=dev)
        self._empty_i = torch.empty(0, dtype=torch.int32, device=dev)
        if weights_dev is None:
            self.init_embedding_weights_uniform(-0.01, 0.01)

    @torch.no_grad()
    def init_embedding_weights_uniform(self, lo: float, hi: float) -> None:
        self.weights_dev.copy_((torch.rand(self.weights_dev.numel(), device=self.weights_dev.device)
                                * (hi - lo) + lo).to(self.weights_dev.dtype))

    def split_embedding_weights(self) -> List[torch.Tensor]:
        """Views of the flat buffer, one [rows, dim] tensor per table."""
        out, pos = [], 0
        for rows, dim in self.embedding_specs:
            out.append(self.weights_dev.detach()[pos:pos + rows * dim].view(rows, dim))
            pos += rows * dim
        return out

    def forward(self, indices: torch.Tensor, offsets: torch.Tensor,
                per_sample_weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        placeholder = self._placeholder.detach().requires_grad_(torch.is_grad_enabled())
        common = (placeholder, self.weights_dev, self._empty_w, self._empty_w, self._empty_i,
                  self.weights_offsets, self.D_offsets, self.total_D, self.max_D, self.hash_size_cumsum,
                  self.total_hash_size_bits, indices, offsets, int(self.pooling_mode), per_sample_weights,
                  None, self._empty_i, False, 0.0, False)
        if self.optimizer == OptimType.EXACT_SGD:
            return torch.ops.fbgemm.split_embedding_codegen_lookup_sgd_function(
                *common, self.learning_rate, int(self.output_dtype))
        return torch.ops.fbgemm.split_embedding_codegen_lookup_rowwise_adagrad_function(
            *common, self.momentum1_dev, self._empty_f, self._empty_i, self.momentum1_offsets, self.eps,
            self.learning_rate, 0.0, 0, 0.0, int(self.output_dtype))


class IntNBitTableBatchedEmbeddingBagsCodegen(torch.nn.Module):
    """Quantised inference tables: embedding_specs is [(rows, dim, SparseType), ...]. Tables are
    filled from float tensors with `assign_table`, which quantises on the GPU."""

    def __init__(self, embedding_specs: Sequence[Tuple[int, int, SparseType]],
                 pooling_mode: PoolingMode = PoolingMode.SUM, output_dtype: SparseType = SparseType.FP16,
                 row_alignment: int = 16, device="cuda"):
        super().__init__()
        load_torch_ops()
        self.embedding_specs = [(int(r), int(d), SparseType(t)) for r, d, t in embedding_specs]
        self.pooling_mode, self.output_dtype = PoolingMode(pooling_mode), SparseType(output_dtype)
        self.row_alignment = int(row_alignment)
        dev = torch.device(device)
        w_off, d_off, pos, strides = [], [0], 0, []
        for rows, dim, ty in self.embedding_specs:
            stride = self.row_bytes(dim, ty)
            pos = _round_up(pos, 16)
            w_off.append(pos)
            strides.append(stride)
            pos += rows * stride
            d_off.append(d_off[-1] + dim)
        self.row_strides = strides
        self.total_D = d_off[-1]
        self.max_D_by_type = {t: max([d for _, d, ty in self.embedding_specs if ty == t], default=0)
                              for t in SparseType}
        self.register_buffer("weights_dev", torch.zeros(pos, dtype=torch.uint8, device=dev))
        self.register_buffer("weights_offsets", torch.tensor(w_off, dtype=torch.int64, device=dev))
        self.register_buffer("weights_tys", torch.tensor([int(t) for _, _, t in self.embedding_specs],
                                                         dtype=torch.uint8, device=dev))
        self.register_buffer("D_offsets", torch.tensor(d_off, dtype=torch.int32, device=dev))
        self._w_off_host = w_off
        self._empty_u8 = torch.empty(0, dtype=torch.uint8, device=dev)
        self._empty_i = torch.empty(0, dtype=torch.int32, device=dev)

    def row_bytes(self, dim: int, ty: SparseType) -> int:
        if ty in (SparseType.INT8, SparseType.INT4, SparseType.INT2):
            return int(cabi.lib().b200tbe_quantized_row_bytes(dim, int(ty), self.row_alignment))
        return _round_up(dim * (2 if ty == SparseType.FP16 else 4), self.row_alignment)

    @torch.no_grad()
    def assign_table(self, t: int, weights: torch.Tensor) -> None:
        """Stores a float [rows, dim] table as table t, quantising it on the GPU when t is an
        integer-typed table."""
        rows, dim, ty = self.embedding_specs[t]
        if tuple(weights.shape) != (rows, dim):
            raise ValueError("table %d is [%d, %d]" % (t, rows, dim))
        stride, start = self.row_strides[t], self._w_off_host[t]
        dst = self.weights_dev[start:start + rows * stride].view(rows, stride)
        src = weights.to(self.weights_dev.device).contiguous()
        if ty in (SparseType.INT8, SparseType.INT4, SparseType.INT2):
            if src.dtype not in (torch.float32, torch.float16):
                src = src.float()
            dst.copy_(cabi.quantize_rows(src, int(ty), self.row_alignment, header_first=True))
        else:
            raw = src.to(torch.float16 if ty == SparseType.FP16 else torch.float32).view(torch.uint8)
            dst.zero_()
            dst[:, :raw.shape[1]] = raw.view(rows, -1)

    def forward(self, indices: torch.Tensor, offsets: torch.Tensor,
                per_sample_weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        m = self.max_D_by_type
        return torch.ops.fbgemm.int_nbit_split_embedding_codegen_lookup_function(
            self.weights_dev, self._empty_u8, self._empty_i, self.weights_offsets, self.weights_tys,
            self.D_offsets, self.total_D, m[SparseType.INT2], m[SparseType.INT4], m[SparseType.INT8],
            m[SparseType.FP16], m[SparseType.FP32], indices, offsets, int(self.pooling_mode),
            per_sample_weights, int(self.output_dtype), None, None, self.row_alignment)
