"""CPU oracle for the TBE / jagged hot path -- TEST INFRASTRUCTURE, not product code.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this package.
Two back ends, both taking and returning numpy arrays:

  * `c`   -- oracle/tbe_oracle.c, a plain-C restatement of the arithmetic (see its header for what
             it follows and how it is pinned; parity against fbgemm_gpu itself is UNPINNED);
  * `ref` -- oracle/fbgemm_core_ref.cpp, the FBGEMM-core CPU kernels that ship inside torch's
             libtorch_cpu.so, used to pin the restatement and as the timed CPU arm.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import build as _build

FP32, FP16, INT8, INT4, INT2 = 0, 1, 2, 3, 4
SUM, MEAN = 0, 1
SGD, ROWWISE_ADAGRAD = 0, 1

_c = None
_ref = None


def _ptr(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(ctypes.c_void_p)


def c_lib():
    global _c
    if _c is None:
        _c = ctypes.CDLL(_build.build_c_oracle())
        _c.oracle_half_to_float.restype = ctypes.c_float
        _c.oracle_half_to_float.argtypes = [ctypes.c_uint16]
        _c.oracle_float_to_half.restype = ctypes.c_uint16
        _c.oracle_float_to_half.argtypes = [ctypes.c_float]
        _c.oracle_nbit_row_stride.restype = ctypes.c_int64
        _c.oracle_nbit_row_stride.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
    return _c


def ref_lib():
    global _ref
    if _ref is None:
        import torch  # noqa: F401  (makes libtorch_cpu.so resident before the harness links to it)

        _ref = ctypes.CDLL(_build.build_fbgemm_core_ref())
    return _ref


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def nbit_row_stride(ty: int, D: int, row_alignment: int) -> int:
    return int(c_lib().oracle_nbit_row_stride(ty, D, row_alignment))


def _total_D(D_offsets):
    return int(D_offsets[-1])


def tbe_forward(dev_weights, weights_ty, weights_offsets, D_offsets, B, indices, offsets,
                per_sample_weights=None, pooling_mode=SUM, backend="c", rows_per_table=None):
    """Pooled lookups over fp32/fp16 tables -> fp32 [B, total_D]."""
    T = len(weights_offsets)
    total_D = _total_D(D_offsets)
    out = np.zeros((B, total_D), dtype=np.float32)
    dev_weights = np.ascontiguousarray(dev_weights)
    assert dev_weights.dtype == (np.float32 if weights_ty == FP32 else np.float16)
    wo, do, idx, off = _i64(weights_offsets), _i32(D_offsets), _i64(indices), _i64(offsets)
    psw = None if per_sample_weights is None else np.ascontiguousarray(per_sample_weights, np.float32)
    if backend == "c":
        rc = c_lib().oracle_tbe_forward(
            _ptr(dev_weights), ctypes.c_int(weights_ty), _ptr(wo), _ptr(do), ctypes.c_int(T),
            ctypes.c_int(B), _ptr(idx), _ptr(off), _ptr(psw), ctypes.c_int(pooling_mode), _ptr(out),
            ctypes.c_int64(total_D))
    else:
        rpt = _i64(rows_per_table)
        rc = ref_lib().ref_tbe_forward(
            _ptr(dev_weights), ctypes.c_int(weights_ty), _ptr(wo), _ptr(do), _ptr(rpt),
            ctypes.c_int(T), ctypes.c_int(B), _ptr(idx), _ptr(off), _ptr(psw),
            ctypes.c_int(pooling_mode), _ptr(out), ctypes.c_int64(total_D))
    if rc != 0:
        raise RuntimeError("oracle tbe_forward failed: %d" % rc)
    return out


def nbit_forward(dev_weights, weights_offsets, weights_tys, D_offsets, row_alignment, B, indices,
                 offsets, per_sample_weights=None, pooling_mode=SUM, backend="c",
                 rows_per_table=None):
    """Pooled lookups over quantised tables (byte buffer) -> fp32 [B, total_D]."""
    T = len(weights_offsets)
    total_D = _total_D(D_offsets)
    out = np.zeros((B, total_D), dtype=np.float32)
    dev_weights = np.ascontiguousarray(dev_weights, dtype=np.uint8)
    wo, do, idx, off = _i64(weights_offsets), _i32(D_offsets), _i64(indices), _i64(offsets)
    tys = np.ascontiguousarray(weights_tys, dtype=np.uint8)
    psw = None if per_sample_weights is None else np.ascontiguousarray(per_sample_weights, np.float32)
    if backend == "c":
        rc = c_lib().oracle_nbit_forward(
            _ptr(dev_weights), _ptr(wo), _ptr(tys), _ptr(do), ctypes.c_int(row_alignment),
            ctypes.c_int(T), ctypes.c_int(B), _ptr(idx), _ptr(off), _ptr(psw),
            ctypes.c_int(pooling_mode), _ptr(out), ctypes.c_int64(total_D))
    else:
        rpt = _i64(rows_per_table)
        rc = ref_lib().ref_nbit_forward(
            _ptr(dev_weights), _ptr(wo), _ptr(tys), _ptr(do), _ptr(rpt),
            ctypes.c_int(row_alignment), ctypes.c_int(T), ctypes.c_int(B), _ptr(idx), _ptr(off),
            _ptr(psw), ctypes.c_int(pooling_mode), _ptr(out), ctypes.c_int64(total_D))
    if rc != 0:
        raise RuntimeError("oracle nbit_forward failed: %d" % rc)
    return out


def quantize_rows(src, ty, row_alignment=16, backend="c"):
    """fp32 [rows, D] -> uint8 [rows, stride] in the header-first TBE row layout."""
    src = np.ascontiguousarray(src, dtype=np.float32)
    rows, D = src.shape
    stride = nbit_row_stride(ty, D, row_alignment)
    dst = np.zeros((rows, stride), dtype=np.uint8)
    fn = c_lib().oracle_quantize_rows if backend == "c" else ref_lib().ref_quantize_rows
    rc = fn(_ptr(src), ctypes.c_int64(rows), ctypes.c_int(D), ctypes.c_int(ty),
            ctypes.c_int(row_alignment), _ptr(dst))
    if rc != 0:
        raise RuntimeError("oracle quantize_rows failed: %d" % rc)
    return dst


def dequantize_rows_ref(rows_u8, D, ty):
    """Header-first rows with stride 4 + payload -> fp32 [rows, D], by FBGEMM-core."""
    rows_u8 = np.ascontiguousarray(rows_u8, dtype=np.uint8)
    out = np.zeros((rows_u8.shape[0], D), dtype=np.float32)
    rc = ref_lib().ref_dequantize_rows(_ptr(rows_u8), ctypes.c_int64(rows_u8.shape[0]),
                                       ctypes.c_int(D), ctypes.c_int(ty), _ptr(out))
    if rc != 0:
        raise RuntimeError("ref_dequantize_rows failed: %d" % rc)
    return out


def tbe_backward(dev_weights, weights_ty, weights_offsets, D_offsets, hash_size_cumsum, B, indices,
                 offsets, grad, momentum1, momentum1_offsets, optimizer, lr, eps,
                 per_sample_weights=None, pooling_mode=SUM):
    """Exact fused backward; dev_weights and momentum1 are updated IN PLACE."""
    T = len(weights_offsets)
    assert dev_weights.flags["C_CONTIGUOUS"] and dev_weights.flags["WRITEABLE"]
    assert dev_weights.dtype == (np.float32 if weights_ty == FP32 else np.float16)
    grad = np.ascontiguousarray(grad, dtype=np.float32)
    wo, do, hs = _i64(weights_offsets), _i32(D_offsets), _i64(hash_size_cumsum)
    idx, off = _i64(indices), _i64(offsets)
    mo = None if momentum1_offsets is None else _i64(momentum1_offsets)
    if momentum1 is not None:
        assert momentum1.dtype == np.float32 and momentum1.flags["C_CONTIGUOUS"]
    psw = None if per_sample_weights is None else np.ascontiguousarray(per_sample_weights, np.float32)
    rc = c_lib().oracle_tbe_backward(
        _ptr(dev_weights), ctypes.c_int(weights_ty), _ptr(wo), _ptr(do), _ptr(hs), ctypes.c_int(T),
        ctypes.c_int(B), _ptr(idx), _ptr(off), _ptr(psw), ctypes.c_int(pooling_mode), _ptr(grad),
        ctypes.c_int64(grad.shape[1]), _ptr(momentum1), _ptr(mo), ctypes.c_int(optimizer),
        ctypes.c_float(lr), ctypes.c_float(eps))
    if rc != 0:
        raise RuntimeError("oracle tbe_backward failed: %d" % rc)


def rowwise_adagrad_fused_ref(w, g, h, indices, offsets, eps, lr):
    """FBGEMM-core's fused row-wise Adagrad reference (per-lookup, not de-duplicated); in place."""
    ty = FP32 if w.dtype == np.float32 else FP16
    rows, D = w.shape
    g = np.ascontiguousarray(g, dtype=np.float32)
    idx, off = _i64(indices), _i64(offsets)
    rc = ref_lib().ref_rowwise_adagrad_fused(
        ctypes.c_int(ty), ctypes.c_int64(D), ctypes.c_int64(len(off) - 1), ctypes.c_int64(len(idx)),
        ctypes.c_int64(rows), _ptr(w), _ptr(g), _ptr(h), _ptr(idx), _ptr(off), ctypes.c_float(eps),
        ctypes.c_float(-lr), ctypes.c_int64(g.shape[1]))
    if rc != 1:  # the reference returns 1 on success, 0 on a malformed input
        raise RuntimeError("ref_rowwise_adagrad_fused failed: %d" % rc)


def _offsets_array(offsets_list):
    keep = [_i64(o) for o in offsets_list]
    arr = (ctypes.c_void_p * len(keep))(*[o.ctypes.data for o in keep])
    return keep, arr


def _dense_shape(outer, max_lengths, inner):
    return (outer, *[int(m) for m in max_lengths], inner)


def jagged_to_padded_dense(values, offsets_list, max_lengths, padding_value=0):
    values = np.ascontiguousarray(values)
    keep, arr = _offsets_array(offsets_list)
    outer = len(keep[0]) - 1
    inner = values.shape[1]
    ml = _i64(max_lengths)
    dense = np.empty(_dense_shape(outer, max_lengths, inner), dtype=values.dtype)
    pad = np.array([padding_value], dtype=values.dtype)
    rc = c_lib().oracle_jagged_to_padded_dense(
        _ptr(values), arr, _ptr(ml), ctypes.c_int(len(keep)), ctypes.c_int64(outer),
        ctypes.c_int64(inner), ctypes.c_int64(values.shape[0]), ctypes.c_int(values.itemsize),
        _ptr(pad), _ptr(dense))
    if rc != 0:
        raise RuntimeError("oracle jagged_to_padded_dense failed: %d" % rc)
    return dense


def dense_to_jagged(dense, offsets_list, total_rows=None):
    dense = np.ascontiguousarray(dense)
    keep, arr = _offsets_array(offsets_list)
    outer = len(keep[0]) - 1
    n = len(keep)
    inner = dense.shape[-1]
    ml = _i64(dense.shape[1:1 + n])
    if total_rows is None:
        total_rows = int(keep[-1][-1])
    values = np.empty((total_rows, inner), dtype=dense.dtype)
    rc = c_lib().oracle_dense_to_jagged(
        _ptr(dense), arr, _ptr(ml), ctypes.c_int(n), ctypes.c_int64(outer), ctypes.c_int64(inner),
        ctypes.c_int64(total_rows), ctypes.c_int(dense.itemsize), _ptr(values))
    if rc != 0:
        raise RuntimeError("oracle dense_to_jagged failed: %d" % rc)
    return values


def jagged_dense_elementwise_add(x_values, offsets_list, y):
    x_values = np.ascontiguousarray(x_values, dtype=np.float32)
    y = np.ascontiguousarray(y, dtype=np.float32)
    keep, arr = _offsets_array(offsets_list)
    outer = len(keep[0]) - 1
    n = len(keep)
    inner = y.shape[-1]
    ml = _i64(y.shape[1:1 + n])
    out = np.empty_like(y)
    rc = c_lib().oracle_jagged_dense_elementwise_add_f32(
        _ptr(x_values), arr, _ptr(ml), ctypes.c_int(n), ctypes.c_int64(outer),
        ctypes.c_int64(inner), ctypes.c_int64(x_values.shape[0]), _ptr(y), _ptr(out))
    if rc != 0:
        raise RuntimeError("oracle jagged_dense_elementwise_add failed: %d" % rc)
    return out


def permute_segments(values, lengths, perm):
    """out segment j = in segment perm[j] (numpy): the data movement of
    torch.ops.fbgemm.permute_2D_sparse_data, restated as an index gather."""
    values, lengths, perm = np.asarray(values), np.asarray(lengths, dtype=np.int64), np.asarray(perm, dtype=np.int64)
    in_off = np.zeros(lengths.size + 1, dtype=np.int64)
    np.cumsum(lengths, out=in_off[1:])
    out_len = lengths[perm]
    out_off = np.zeros(perm.size + 1, dtype=np.int64)
    np.cumsum(out_len, out=out_off[1:])
    src = np.arange(int(out_off[-1]), dtype=np.int64) + np.repeat(in_off[:-1][perm] - out_off[:-1], out_len)
    return values[src]


def num_threads() -> int:
    return int(ref_lib().ref_num_threads())


def set_num_threads(n: int) -> int:
    """Thread count of both oracle libraries from here on (they share one OpenMP runtime), whatever
    OMP_NUM_THREADS the launcher exported. Returns the count in effect."""
    c_lib()
    ref_lib().ref_set_num_threads(ctypes.c_int(int(n)))
    return num_threads()


# ---- NV12 -> RGB24 (nv12_oracle.c) ----------------------------------------------------------
_nv12 = None


def nv12_lib():
    global _nv12
    if _nv12 is None:
        _nv12 = ctypes.CDLL(_build.build_nv12_oracle())
        _nv12.nv12_oracle_offset.restype = ctypes.c_size_t
        _nv12.nv12_oracle_offset.argtypes = [ctypes.c_int] * 4
        _nv12.nv12_oracle_pixel.restype = None
        _nv12.nv12_oracle_pixel.argtypes = [ctypes.c_uint8] * 3 + [ctypes.c_int, ctypes.c_void_p]
        _nv12.nv12_oracle_convert.restype = None
        _nv12.nv12_oracle_convert.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 5
    return _nv12


def nv12_all_triples(fullrange: bool = False) -> np.ndarray:
    """RGB of every (y, u, v) triple: uint8 [256, 256, 256, 3]."""
    out = np.zeros((256, 256, 256, 3), dtype=np.uint8)
    lib = nv12_lib()
    lib.nv12_oracle_all_triples.restype = None
    lib.nv12_oracle_all_triples.argtypes = [ctypes.c_int, ctypes.c_void_p]
    lib.nv12_oracle_all_triples(int(fullrange), _ptr(out))
    return out


class Nv12Reference:
    """The reference's ColorConversionKernel.cpp compiled for the host (oracle/_ref, built by
    oracle/build.py where the reference tree is present). contracted=True: the build that lets the
    compiler fuse the dot products' multiply-adds."""

    def __init__(self, contracted: bool = False):
        libs = _build.build_nv12_reference()
        name = "nv12_ref_fma" if contracted else "nv12_ref"
        if name not in libs:
            raise FileNotFoundError("oracle/_ref/lib%s.so is not built (no reference tree here)" % name)
        self.lib = ctypes.CDLL(libs[name])
        self.lib.nv12_ref_tile_offset.restype = ctypes.c_size_t
        self.lib.nv12_ref_tile_offset.argtypes = [ctypes.c_int] * 3
        self.lib.nv12_ref_all_triples.restype = None
        self.lib.nv12_ref_all_triples.argtypes = [ctypes.c_int, ctypes.c_void_p]
        self.lib.nv12_ref_convert.restype = None
        self.lib.nv12_ref_convert.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 4

    def tile_offset(self, x: int, y: int, stride: int) -> int:
        return int(self.lib.nv12_ref_tile_offset(x, y, stride))

    def all_triples(self, fullrange: bool = False) -> np.ndarray:
        out = np.zeros((256, 256, 256, 3), dtype=np.uint8)
        self.lib.nv12_ref_all_triples(int(fullrange), _ptr(out))
        return out

    def convert(self, y_plane, uv_plane, width, height, stride, fullrange=False) -> np.ndarray:
        y_plane = np.ascontiguousarray(y_plane, dtype=np.uint8)
        uv_plane = np.ascontiguousarray(uv_plane, dtype=np.uint8)
        rgb = np.zeros((height, width, 3), dtype=np.uint8)
        self.lib.nv12_ref_convert(_ptr(y_plane), _ptr(uv_plane), _ptr(rgb), width, height, stride, int(fullrange))
        return rgb


def nv12_offset(x: int, y: int, stride: int, tiled: bool) -> int:
    return int(nv12_lib().nv12_oracle_offset(x, y, stride, int(tiled)))


def nv12_pixel(y: int, u: int, v: int, fullrange: bool = False):
    out = np.zeros(3, dtype=np.uint8)
    nv12_lib().nv12_oracle_pixel(y, u, v, int(fullrange), _ptr(out))
    return tuple(int(c) for c in out)


def nv12_to_rgb(y_plane, uv_plane, width: int, height: int, stride: int, fullrange: bool = False,
                tiled: bool = False):
    """y_plane / uv_plane: contiguous uint8 arrays (surface bytes); returns [height, width, 3] uint8."""
    y_plane = np.ascontiguousarray(y_plane, dtype=np.uint8)
    uv_plane = np.ascontiguousarray(uv_plane, dtype=np.uint8)
    rgb = np.empty((height, width, 3), dtype=np.uint8)
    nv12_lib().nv12_oracle_convert(_ptr(y_plane), _ptr(uv_plane), _ptr(rgb), width, height, stride,
                                   int(fullrange), int(tiled))
    return rgb
