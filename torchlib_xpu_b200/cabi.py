"""ctypes binding of the C ABI in include/b200tbe.h.

The structures below mirror the header field by field. The helper functions take torch CUDA tensors
only to read their data pointers and the current stream; every computation happens in
libb200tbe.so. There is no fallback: if the library is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _build

MAX_DESTS = 16
MAX_JAGGED_DIMS = 4

FP32, FP16, INT8, INT4, INT2, BF16 = 0, 1, 2, 3, 4, 5
POOL_SUM, POOL_MEAN, POOL_NONE = 0, 1, 2
OPT_SGD, OPT_ROWWISE_ADAGRAD = 0, 1
DEV_INDEX_OUT_OF_RANGE = 1

_c_void_p = ctypes.c_void_p


class ForwardParams(ctypes.Structure):
    _fields_ = [
        ("dev_weights", _c_void_p), ("weights_offsets", _c_void_p), ("D_offsets", _c_void_p),
        ("rows_per_table", _c_void_p), ("indices", _c_void_p), ("offsets", _c_void_p),
        ("per_sample_weights", _c_void_p), ("outputs", _c_void_p * MAX_DESTS),
        ("output_stride", ctypes.c_int64), ("output_col_offset", ctypes.c_int64),
        ("rows_per_dest", ctypes.c_int64), ("num_dests", ctypes.c_int32), ("T", ctypes.c_int32),
        ("B", ctypes.c_int32), ("max_D", ctypes.c_int32), ("weights_dtype", ctypes.c_int32),
        ("output_dtype", ctypes.c_int32), ("index_bytes", ctypes.c_int32),
        ("pooling_mode", ctypes.c_int32), ("status", _c_void_p),
    ]


class NbitForwardParams(ctypes.Structure):
    _fields_ = [
        ("dev_weights", _c_void_p), ("weights_offsets", _c_void_p), ("weights_tys", _c_void_p),
        ("D_offsets", _c_void_p), ("rows_per_table", _c_void_p), ("indices", _c_void_p),
        ("offsets", _c_void_p), ("per_sample_weights", _c_void_p),
        ("outputs", _c_void_p * MAX_DESTS), ("output_stride", ctypes.c_int64),
        ("output_col_offset", ctypes.c_int64), ("rows_per_dest", ctypes.c_int64),
        ("num_dests", ctypes.c_int32), ("T", ctypes.c_int32), ("B", ctypes.c_int32),
        ("max_D", ctypes.c_int32), ("row_alignment", ctypes.c_int32),
        ("output_dtype", ctypes.c_int32), ("index_bytes", ctypes.c_int32),
        ("pooling_mode", ctypes.c_int32), ("status", _c_void_p), ("table_type_mask", ctypes.c_uint32),
    ]


class BackwardParams(ctypes.Structure):
    _fields_ = [
        ("dev_weights", _c_void_p), ("weights_offsets", _c_void_p), ("D_offsets", _c_void_p),
        ("hash_size_cumsum", _c_void_p), ("indices", _c_void_p), ("offsets", _c_void_p),
        ("per_sample_weights", _c_void_p), ("grad_output", _c_void_p),
        ("grad_stride", ctypes.c_int64), ("grad_col_offset", ctypes.c_int64),
        ("momentum1", _c_void_p), ("momentum1_offsets", _c_void_p),
        ("num_indices", ctypes.c_int64), ("T", ctypes.c_int32), ("B", ctypes.c_int32),
        ("max_D", ctypes.c_int32), ("total_hash_size_bits", ctypes.c_int32),
        ("weights_dtype", ctypes.c_int32), ("grad_dtype", ctypes.c_int32),
        ("index_bytes", ctypes.c_int32), ("pooling_mode", ctypes.c_int32),
        ("optimizer", ctypes.c_int32), ("learning_rate", ctypes.c_float), ("eps", ctypes.c_float),
        ("scratch", _c_void_p), ("scratch_bytes", ctypes.c_size_t), ("status", _c_void_p),
        ("grad_ready_event", _c_void_p), ("max_table_rows", ctypes.c_int64),
    ]


class ExchangePushParams(ctypes.Structure):
    _fields_ = [
        ("src", _c_void_p), ("dsts", _c_void_p * MAX_DESTS), ("src_stride_bytes", ctypes.c_int64),
        ("dst_stride_bytes", ctypes.c_int64), ("dst_row_offset", ctypes.c_int64), ("rows", ctypes.c_int64),
        ("block_bytes", ctypes.c_int64), ("num_dsts", ctypes.c_int32),
    ]


class JaggedShape(ctypes.Structure):
    _fields_ = [
        ("offsets", _c_void_p * MAX_JAGGED_DIMS), ("max_lengths", ctypes.c_int64 * MAX_JAGGED_DIMS),
        ("num_jagged_dims", ctypes.c_int32), ("offset_bytes", ctypes.c_int32),
        ("outer_size", ctypes.c_int64), ("inner_size", ctypes.c_int64),
        ("total_rows", ctypes.c_int64), ("elem_bytes", ctypes.c_int32), ("dtype", ctypes.c_int32),
    ]


# Every symbol include/b200tbe.h declares; tests check that the library exports all of them.
EXPORTS = (
    "b200tbe_status_string", "b200tbe_abi_version", "b200tbe_forward", "b200tbe_nbit_forward",
    "b200tbe_backward_scratch_bytes", "b200tbe_backward", "b200tbe_radix_sort_scratch_bytes",
    "b200tbe_radix_sort_pairs", "b200tbe_radix_sort_segments_scratch_bytes",
    "b200tbe_radix_sort_segments", "b200tbe_radix_sort_pairs_static_max",
    "b200tbe_radix_sort_pairs_static", "b200tbe_exchange_push", "b200tbe_permute_segments", "b200tbe_quantized_row_bytes",
    "b200tbe_quantize_rows", "b200tbe_dequantize_rows", "b200tbe_nv12_to_rgb", "b200tbe_jagged_to_padded_dense", "b200tbe_dense_to_jagged",
    "b200tbe_jagged_dense_elementwise_add",
)

_lib = None


def library_path() -> str:
    return _build.CABI_LIB


def lib() -> ctypes.CDLL:
    """Loads libb200tbe.so (built in-tree beforehand). Raises if it is missing: there is no other
    implementation to fall back to."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                "libb200tbe.so is not built (%s). Run `python -m torchlib_xpu_b200._build`; "
                "the CUDA kernels are the only implementation of this package." % path)
        _lib = ctypes.CDLL(path)
        _lib.b200tbe_status_string.restype = ctypes.c_char_p
        _lib.b200tbe_status_string.argtypes = [ctypes.c_int]
        _lib.b200tbe_backward_scratch_bytes.restype = ctypes.c_size_t
        _lib.b200tbe_backward_scratch_bytes.argtypes = [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32,
                                                        ctypes.c_int32]
        _lib.b200tbe_radix_sort_scratch_bytes.restype = ctypes.c_size_t
        _lib.b200tbe_radix_sort_scratch_bytes.argtypes = [ctypes.c_int64]
        _lib.b200tbe_radix_sort_pairs.argtypes = [
            _c_void_p, _c_void_p, _c_void_p, _c_void_p, ctypes.c_int64, ctypes.c_int32,
            ctypes.c_int32, _c_void_p, ctypes.c_size_t, _c_void_p]
        _lib.b200tbe_radix_sort_segments_scratch_bytes.restype = ctypes.c_size_t
        _lib.b200tbe_radix_sort_segments_scratch_bytes.argtypes = [ctypes.c_int64, ctypes.c_int32]
        _lib.b200tbe_radix_sort_segments.argtypes = [
            _c_void_p, _c_void_p, _c_void_p, _c_void_p, ctypes.c_int64, _c_void_p, ctypes.c_int32,
            ctypes.c_int32, ctypes.c_int32, _c_void_p, ctypes.c_size_t, _c_void_p]
        _lib.b200tbe_radix_sort_pairs_static_max.restype = ctypes.c_int64
        _lib.b200tbe_radix_sort_pairs_static_max.argtypes = []
        _lib.b200tbe_radix_sort_pairs_static.argtypes = [
            _c_void_p, _c_void_p, _c_void_p, _c_void_p, ctypes.c_int64, ctypes.c_int32,
            ctypes.c_int32, _c_void_p]
        _lib.b200tbe_exchange_push.argtypes = [ctypes.POINTER(ExchangePushParams), _c_void_p]
        _lib.b200tbe_permute_segments.argtypes = [_c_void_p] * 5 + [ctypes.c_int64, ctypes.c_int64] + \
            [ctypes.c_int32] * 3 + [_c_void_p]
        _lib.b200tbe_quantized_row_bytes.restype = ctypes.c_int64
        _lib.b200tbe_quantized_row_bytes.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
        _lib.b200tbe_quantize_rows.argtypes = [
            _c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
            ctypes.c_int32, _c_void_p, _c_void_p]
        _lib.b200tbe_dequantize_rows.argtypes = [
            _c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
            _c_void_p, ctypes.c_int32, _c_void_p]
        _lib.b200tbe_nv12_to_rgb.argtypes = [_c_void_p, _c_void_p, _c_void_p] + [ctypes.c_int32] * 5 + [_c_void_p]
        _lib.b200tbe_forward.argtypes = [ctypes.POINTER(ForwardParams), _c_void_p]
        _lib.b200tbe_nbit_forward.argtypes = [ctypes.POINTER(NbitForwardParams), _c_void_p]
        _lib.b200tbe_backward.argtypes = [ctypes.POINTER(BackwardParams), _c_void_p]
        _lib.b200tbe_jagged_to_padded_dense.argtypes = [
            ctypes.POINTER(JaggedShape), _c_void_p, _c_void_p, ctypes.c_uint64, _c_void_p]
        _lib.b200tbe_dense_to_jagged.argtypes = [
            ctypes.POINTER(JaggedShape), _c_void_p, _c_void_p, _c_void_p]
        _lib.b200tbe_jagged_dense_elementwise_add.argtypes = [
            ctypes.POINTER(JaggedShape), _c_void_p, _c_void_p, _c_void_p, _c_void_p]
    return _lib


class B200TbeError(RuntimeError):
    pass


def check(status: int, what: str) -> None:
    if status != 0:
        raise B200TbeError("%s: %s (%d)" % (what, lib().b200tbe_status_string(status).decode(), status))


def _p(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise B200TbeError("b200tbe entry points take CUDA tensors only")
    if not t.is_contiguous():
        raise B200TbeError("b200tbe entry points take contiguous tensors")
    return t.data_ptr() or None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_TORCH_TO_CODE = {torch.float32: FP32, torch.float16: FP16, torch.bfloat16: BF16}
_CODE_TO_TORCH = {FP32: torch.float32, FP16: torch.float16, BF16: torch.bfloat16}


def _index_bytes(indices, offsets) -> int:
    if indices.dtype != offsets.dtype or indices.dtype not in (torch.int64, torch.int32):
        raise B200TbeError("indices and offsets must both be int64 or both int32")
    return indices.element_size()


def forward(dev_weights, weights_offsets, D_offsets, total_D, max_D, indices, offsets, B,
            pooling_mode=POOL_SUM, per_sample_weights=None, output_dtype=torch.float32,
            rows_per_table=None, status=None, outputs=None, output_stride=None,
            output_col_offset=0, rows_per_dest=None):
    """b200tbe_forward over torch tensors. Returns the [B, total_D] output (or `outputs` when the
    caller supplies destination buffers)."""
    T = weights_offsets.numel()
    p = ForwardParams()
    p.dev_weights, p.weights_offsets, p.D_offsets = _p(dev_weights), _p(weights_offsets), _p(D_offsets)
    p.rows_per_table, p.indices, p.offsets = _p(rows_per_table), _p(indices), _p(offsets)
    p.per_sample_weights = _p(per_sample_weights)
    result = None
    if outputs is None:
        result = torch.empty((B, total_D), dtype=output_dtype, device=dev_weights.device)
        outputs = [result]
        output_stride, rows_per_dest = total_D, max(B, 1)
    for i, o in enumerate(outputs):
        p.outputs[i] = o if isinstance(o, int) else _p(o)
    p.output_stride, p.output_col_offset, p.rows_per_dest = output_stride, output_col_offset, rows_per_dest
    p.num_dests, p.T, p.B, p.max_D = len(outputs), T, B, max_D
    p.weights_dtype = _TORCH_TO_CODE[dev_weights.dtype]
    p.output_dtype = _TORCH_TO_CODE[output_dtype]
    p.index_bytes = _index_bytes(indices, offsets)
    p.pooling_mode = pooling_mode
    p.status = _p(status)
    check(lib().b200tbe_forward(ctypes.byref(p), _stream()), "b200tbe_forward")
    return result if result is not None else outputs


def nbit_forward(dev_weights, weights_offsets, weights_tys, D_offsets, total_D, max_D, indices,
                 offsets, B, pooling_mode=POOL_SUM, per_sample_weights=None,
                 output_dtype=torch.float16, row_alignment=16, rows_per_table=None, status=None,
                 table_types=None):
    """b200tbe_nbit_forward over torch tensors. table_types: the type codes present among the tables
    (any iterable of ints), when the caller knows them on the host; None: unknown."""
    T = weights_offsets.numel()
    p = NbitForwardParams()
    p.dev_weights, p.weights_offsets, p.weights_tys = _p(dev_weights), _p(weights_offsets), _p(weights_tys)
    p.D_offsets, p.rows_per_table = _p(D_offsets), _p(rows_per_table)
    p.indices, p.offsets, p.per_sample_weights = _p(indices), _p(offsets), _p(per_sample_weights)
    out = torch.empty((B, total_D), dtype=output_dtype, device=dev_weights.device)
    p.outputs[0] = _p(out)
    p.output_stride, p.output_col_offset, p.rows_per_dest = total_D, 0, max(B, 1)
    p.num_dests, p.T, p.B, p.max_D = 1, T, B, max_D
    p.row_alignment = row_alignment
    p.output_dtype = _TORCH_TO_CODE[output_dtype]
    p.index_bytes = _index_bytes(indices, offsets)
    p.pooling_mode = pooling_mode
    p.status = _p(status)
    p.table_type_mask = 0
    for code in (table_types or ()):
        p.table_type_mask |= 1 << int(code)
    check(lib().b200tbe_nbit_forward(ctypes.byref(p), _stream()), "b200tbe_nbit_forward")
    return out


def backward_scratch_bytes(num_indices: int, total_hash_size_bits: int, max_D: int, T: int) -> int:
    return int(lib().b200tbe_backward_scratch_bytes(num_indices, total_hash_size_bits, max_D, T))


def backward(dev_weights, weights_offsets, D_offsets, hash_size_cumsum, total_hash_size_bits, max_D,
             indices, offsets, B, grad_output, optimizer, learning_rate, eps=0.0, momentum1=None,
             momentum1_offsets=None, pooling_mode=POOL_SUM, per_sample_weights=None, scratch=None,
             status=None, grad_col_offset=0, grad_ready_event=None, max_table_rows=0):
    """b200tbe_backward over torch tensors; dev_weights and momentum1 are updated in place.
    max_table_rows (rows of the largest table, 0 = unknown) lets the sort skip the key bits that
    only tell tables apart."""
    T = weights_offsets.numel()
    n = indices.numel()
    need = backward_scratch_bytes(n, total_hash_size_bits, max_D, T)
    if scratch is None:
        scratch = torch.empty(max(need, 256), dtype=torch.uint8, device=dev_weights.device)
    p = BackwardParams()
    p.dev_weights, p.weights_offsets, p.D_offsets = _p(dev_weights), _p(weights_offsets), _p(D_offsets)
    p.hash_size_cumsum, p.indices, p.offsets = _p(hash_size_cumsum), _p(indices), _p(offsets)
    p.per_sample_weights, p.grad_output = _p(per_sample_weights), _p(grad_output)
    p.grad_stride, p.grad_col_offset = grad_output.stride(0), grad_col_offset
    p.momentum1, p.momentum1_offsets = _p(momentum1), _p(momentum1_offsets)
    p.num_indices, p.T, p.B, p.max_D = n, T, B, max_D
    p.total_hash_size_bits = total_hash_size_bits
    p.weights_dtype = _TORCH_TO_CODE[dev_weights.dtype]
    p.grad_dtype = _TORCH_TO_CODE[grad_output.dtype]
    p.index_bytes = _index_bytes(indices, offsets)
    p.pooling_mode, p.optimizer = pooling_mode, optimizer
    p.learning_rate, p.eps = learning_rate, eps
    p.scratch, p.scratch_bytes = _p(scratch), scratch.numel()
    p.status = _p(status)
    # a recorded torch.cuda.Event: the gradient matrix is complete once it has fired
    p.grad_ready_event = grad_ready_event.cuda_event if grad_ready_event is not None else None
    p.max_table_rows = int(max_table_rows)
    check(lib().b200tbe_backward(ctypes.byref(p), _stream()), "b200tbe_backward")
    return scratch


def radix_sort_pairs(keys, vals, key_bits):
    """Stable sort of (keys, vals) by the low key_bits bits. keys int32/int64, vals int32.
    Returns new (keys, vals); the inputs are clobbered."""
    n = keys.numel()
    keys_out, vals_out = torch.empty_like(keys), torch.empty_like(vals)
    need = int(lib().b200tbe_radix_sort_scratch_bytes(n))
    scratch = torch.empty(max(need, 256), dtype=torch.uint8, device=keys.device)
    check(lib().b200tbe_radix_sort_pairs(_p(keys), _p(vals), _p(keys_out), _p(vals_out), n,
                                         keys.element_size(), key_bits, _p(scratch),
                                         scratch.numel(), _stream()), "b200tbe_radix_sort_pairs")
    return keys_out, vals_out


def radix_sort_segments(keys, vals, seg_offsets, key_bits):
    """Stable sort of every segment [seg_offsets[s], seg_offsets[s+1]) of (keys, vals) by the low
    key_bits bits. keys and vals int32; seg_offsets int32/int64 on the device. Returns new
    (keys, vals); the inputs are clobbered."""
    n = keys.numel()
    num_segments = seg_offsets.numel() - 1
    keys_out, vals_out = torch.empty_like(keys), torch.empty_like(vals)
    need = int(lib().b200tbe_radix_sort_segments_scratch_bytes(n, num_segments))
    scratch = torch.empty(max(need, 256), dtype=torch.uint8, device=keys.device)
    check(lib().b200tbe_radix_sort_segments(_p(keys), _p(vals), _p(keys_out), _p(vals_out), n,
                                            _p(seg_offsets), seg_offsets.element_size(), num_segments,
                                            key_bits, _p(scratch), scratch.numel(), _stream()),
          "b200tbe_radix_sort_segments")
    return keys_out, vals_out


def exchange_push(src, dst_ptrs, dst_stride_bytes, dst_row_offset, block_bytes):
    """b200tbe_exchange_push: src is a [rows, len(dst_ptrs) * block] tensor, dst_ptrs raw device
    addresses of the destinations' matrices (peer-mapped buffers)."""
    p = ExchangePushParams()
    p.src = _p(src)
    for i, ptr in enumerate(dst_ptrs):
        p.dsts[i] = int(ptr)
    p.src_stride_bytes = src.stride(0) * src.element_size()
    p.dst_stride_bytes, p.dst_row_offset = dst_stride_bytes, dst_row_offset
    p.rows, p.block_bytes, p.num_dsts = src.shape[0], block_bytes, len(dst_ptrs)
    check(lib().b200tbe_exchange_push(ctypes.byref(p), _stream()), "b200tbe_exchange_push")


def permute_segments(values, in_offsets, out_offsets, perm):
    """b200tbe_permute_segments: out segment j = in segment perm[j]; values is a flat tensor of 2-,
    4- or 8-byte elements, the offsets int32/int64 tensors of num_segments + 1 entries."""
    out = torch.empty_like(values)
    n = perm.numel()
    check(lib().b200tbe_permute_segments(_p(values), _p(out), _p(in_offsets), _p(out_offsets), _p(perm), n,
                                         values.numel(), values.element_size(), in_offsets.element_size(),
                                         perm.element_size(), _stream()),
          "b200tbe_permute_segments")
    return out


def quantize_rows(src, ty, row_alignment=16, header_first=True, out=None):
    """fp32/fp16 [rows, D] -> uint8 [rows, stride] row-wise quantised (b200tbe_quantize_rows)."""
    rows, D = src.shape
    stride = int(lib().b200tbe_quantized_row_bytes(D, ty, row_alignment))
    if stride < 0:
        raise B200TbeError("unsupported quantised type %r" % (ty,))
    dst = torch.empty((rows, stride), dtype=torch.uint8, device=src.device) if out is None else out
    if dst.shape != (rows, stride) or dst.dtype != torch.uint8 or not dst.is_contiguous():
        raise B200TbeError("out must be a contiguous uint8 [rows, %d] tensor" % stride)
    check(lib().b200tbe_quantize_rows(_p(src), _TORCH_TO_CODE[src.dtype], rows, D, ty, row_alignment,
                                      int(header_first), _p(dst), _stream()), "b200tbe_quantize_rows")
    return dst


def dequantize_rows(rows_u8, D, ty, row_alignment=16, header_first=True, dtype=torch.float32, out=None):
    """uint8 [rows, stride] -> fp32/fp16 [rows, D] (b200tbe_dequantize_rows)."""
    rows = rows_u8.shape[0]
    if out is None:
        out = torch.empty((rows, D), dtype=dtype, device=rows_u8.device)
    elif out.shape != (rows, D) or out.dtype != dtype or not out.is_contiguous():
        raise B200TbeError("out must be a contiguous [rows, D] tensor of the requested dtype")
    check(lib().b200tbe_dequantize_rows(_p(rows_u8), rows, D, ty, row_alignment, int(header_first),
                                        _p(out), _TORCH_TO_CODE[dtype], _stream()),
          "b200tbe_dequantize_rows")
    return out


def nv12_to_rgb(y_plane, uv_plane, width, height, stride, fullrange=False, tiled=False, out=None):
    """NV12 surface (uint8 CUDA tensors holding the luma and the interleaved chroma plane, `stride`
    bytes per row, linear pitch or Intel Tile-Y) -> [height, width, 3] uint8 RGB, BT.709
    (b200tbe_nv12_to_rgb; the reference's convertNV12ToRGB)."""
    if y_plane.dtype != torch.uint8 or uv_plane.dtype != torch.uint8:
        raise B200TbeError("planes must be uint8")
    if out is None:
        out = torch.empty((height, width, 3), dtype=torch.uint8, device=y_plane.device)
    check(lib().b200tbe_nv12_to_rgb(_p(y_plane), _p(uv_plane), _p(out), width, height, stride,
                                    int(bool(fullrange)), int(bool(tiled)), _stream()),
          "b200tbe_nv12_to_rgb")
    return out


def _jagged_shape(offsets_list, max_lengths, outer, inner, total_rows, elem_bytes, dtype_code):
    if not 1 <= len(offsets_list) <= MAX_JAGGED_DIMS or len(offsets_list) != len(max_lengths):
        raise B200TbeError("1..%d jagged dimensions with one max_length each" % MAX_JAGGED_DIMS)
    s = JaggedShape()
    ob = offsets_list[0].element_size()
    for d, (o, m) in enumerate(zip(offsets_list, max_lengths)):
        if o.dtype not in (torch.int64, torch.int32) or o.element_size() != ob:
            raise B200TbeError("offsets must all be int64 or all int32")
        s.offsets[d] = _p(o)
        s.max_lengths[d] = int(m)
    s.num_jagged_dims, s.offset_bytes = len(offsets_list), ob
    s.outer_size, s.inner_size, s.total_rows = outer, inner, total_rows
    s.elem_bytes, s.dtype = elem_bytes, dtype_code
    return s


def _pad_bits(value, dtype) -> int:
    t = torch.tensor([value], dtype=dtype)
    raw = t.view(torch.uint8).tolist()
    return int.from_bytes(bytes(raw), "little")


def jagged_to_padded_dense(values, offsets_list, max_lengths, padding_value=0.0):
    outer = offsets_list[0].numel() - 1
    inner = values.shape[1]
    s = _jagged_shape(offsets_list, max_lengths, outer, inner, values.shape[0],
                      values.element_size(), _TORCH_TO_CODE.get(values.dtype, -1))
    dense = torch.empty((outer, *[int(m) for m in max_lengths], inner), dtype=values.dtype,
                        device=values.device)
    check(lib().b200tbe_jagged_to_padded_dense(ctypes.byref(s), _p(values), _p(dense),
                                               _pad_bits(padding_value, values.dtype), _stream()),
          "b200tbe_jagged_to_padded_dense")
    return dense


def dense_to_jagged(dense, offsets_list, total_rows):
    n = len(offsets_list)
    outer, inner = dense.shape[0], dense.shape[-1]
    s = _jagged_shape(offsets_list, dense.shape[1:1 + n], outer, inner, total_rows,
                      dense.element_size(), _TORCH_TO_CODE.get(dense.dtype, -1))
    values = torch.empty((total_rows, inner), dtype=dense.dtype, device=dense.device)
    check(lib().b200tbe_dense_to_jagged(ctypes.byref(s), _p(dense), _p(values), _stream()),
          "b200tbe_dense_to_jagged")
    return values


def jagged_dense_elementwise_add(x_values, offsets_list, y):
    n = len(offsets_list)
    outer, inner = y.shape[0], y.shape[-1]
    if x_values.dtype != y.dtype or x_values.dtype not in _TORCH_TO_CODE:
        raise B200TbeError("jagged_dense_elementwise_add takes fp32, fp16 or bf16 of one dtype")
    s = _jagged_shape(offsets_list, y.shape[1:1 + n], outer, inner, x_values.shape[0],
                      y.element_size(), _TORCH_TO_CODE[y.dtype])
    out = torch.empty_like(y)
    check(lib().b200tbe_jagged_dense_elementwise_add(ctypes.byref(s), _p(x_values), _p(y), _p(out),
                                                     _stream()),
          "b200tbe_jagged_dense_elementwise_add")
    return out
