// Jagged <-> padded-dense copies and the jagged + dense add.
//
// All three kernels are HBM-bound streaming copies. A CTA owns a tile of consecutive rows of the
// side it iterates over. The first phase resolves, once per row, which row of the other side it
// pairs with (a walk down the offsets levels, or a binary search over offsets) and parks the answer
// in shared memory; the second phase moves the tile with the widest vector the row size and the
// pointers allow (16 bytes in the usual case), four independent loads in flight per thread, fully
// coalesced on the side that is iterated and row-contiguous on the other side.
#include "common.cuh"

namespace b200tbe {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;
constexpr int kMaxRowsPerCta = 256;
constexpr int kTileVecs = kThreads * kUnroll * 2;  // vectors a CTA aims to move

struct JaggedDev {
  const void* offsets[B200TBE_MAX_JAGGED_DIMS];
  int64_t max_lengths[B200TBE_MAX_JAGGED_DIMS];
  int32_t n;
  int64_t total_rows;
};

// Row of `values` that dense row `dense_row` reads, or -1 when the position lies past a length
// (or past the end of values, which malformed offsets could produce).
template <typename OffT>
__device__ __forceinline__ int64_t jagged_row_of(const JaggedDev& s, int64_t dense_row) {
  int64_t coord[B200TBE_MAX_JAGGED_DIMS];
  int64_t r = dense_row;
#pragma unroll
  for (int d = B200TBE_MAX_JAGGED_DIMS - 1; d >= 0; --d) {
    if (d < s.n) {
      coord[d] = r % s.max_lengths[d];
      r /= s.max_lengths[d];
    }
  }
  int64_t idx = r;
#pragma unroll
  for (int d = 0; d < B200TBE_MAX_JAGGED_DIMS; ++d) {
    if (d < s.n) {
      const OffT* off = reinterpret_cast<const OffT*>(s.offsets[d]);
      const int64_t begin = static_cast<int64_t>(__ldg(off + idx));
      const int64_t end = static_cast<int64_t>(__ldg(off + idx + 1));
      if (coord[d] >= end - begin) return -1;
      idx = begin + coord[d];
    }
  }
  return idx < s.total_rows ? idx : -1;
}

template <typename VecT>
__device__ __forceinline__ VecT load_stream(const VecT* p) {
  return __ldcs(p);
}
template <>
__device__ __forceinline__ uint4 load_stream<uint4>(const uint4* p) {
  return ldg_stream16(p);
}
template <typename VecT>
__device__ __forceinline__ void store_stream(VecT* p, VecT v) {
  __stcs(p, v);
}
template <>
__device__ __forceinline__ void store_stream<uint4>(uint4* p, uint4 v) {
  stg_stream16(p, v);
}

template <typename VecT>
__device__ __forceinline__ VecT zero_vec() {
  VecT z;
  memset(&z, 0, sizeof(VecT));
  return z;
}

__device__ __forceinline__ float elem_to_float(float v) { return v; }
__device__ __forceinline__ float elem_to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float elem_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename E>
__device__ __forceinline__ E float_to_elem(float v);
template <>
__device__ __forceinline__ float float_to_elem<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ __half float_to_elem<__half>(float v) {
  return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 float_to_elem<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// a + b element by element. 16-bit types go through fp32 and one rounding, which is what a CPU
// add of the same type produces.
template <typename E, typename VecT>
__device__ __forceinline__ VecT add_elems(VecT a, VecT b) {
  constexpr int kN = sizeof(VecT) / sizeof(E);
  E ea[kN], eb[kN];
  memcpy(ea, &a, sizeof(VecT));
  memcpy(eb, &b, sizeof(VecT));
#pragma unroll
  for (int i = 0; i < kN; ++i) ea[i] = float_to_elem<E>(elem_to_float(ea[i]) + elem_to_float(eb[i]));
  VecT out;
  memcpy(&out, ea, sizeof(VecT));
  return out;
}

enum Mode { kToDense = 0, kFromDense = 1 };

// Iterates over dense rows. kToDense: dense[r] = values[src(r)] or pad. kFromDense:
// values[src(r)] = dense[r] where src(r) exists.
template <typename VecT, typename OffT, int kMode>
__global__ void __launch_bounds__(kThreads)
    jagged_dense_rows_kernel(JaggedDev s, const VecT* __restrict__ src, VecT* __restrict__ dst,
                             VecT pad, int64_t num_dense_rows, uint32_t vecs_per_row,
                             int rows_per_cta) {
  __shared__ int64_t pair_row[kMaxRowsPerCta];
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * rows_per_cta;
  const int64_t left = num_dense_rows - row0;
  const int nrows = left < rows_per_cta ? static_cast<int>(left) : rows_per_cta;
  for (int t = threadIdx.x; t < nrows; t += kThreads) pair_row[t] = jagged_row_of<OffT>(s, row0 + t);
  __syncthreads();

  const uint32_t nvec = static_cast<uint32_t>(nrows) * vecs_per_row;
  const int64_t dense_base = row0 * vecs_per_row;
  for (uint32_t i0 = threadIdx.x; i0 < nvec; i0 += kThreads * kUnroll) {
    VecT v[kUnroll];
    int64_t other[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = i0 + u * kThreads;
      other[u] = -1;
      if (i < nvec) {
        const uint32_t r = i / vecs_per_row;
        const uint32_t c = i - r * vecs_per_row;
        const int64_t pr = pair_row[r];
        if (pr >= 0) other[u] = pr * vecs_per_row + c;
        if (kMode == kToDense) {
          v[u] = pr >= 0 ? load_stream(src + other[u]) : pad;
        } else if (pr >= 0) {
          v[u] = load_stream(src + dense_base + i);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = i0 + u * kThreads;
      if (i < nvec) {
        if (kMode == kToDense) {
          store_stream(dst + dense_base + i, v[u]);
        } else if (other[u] >= 0) {
          store_stream(dst + other[u], v[u]);
        }
      }
    }
  }
}

// out[r] = y[r] + (values[src(r)] or 0), iterating over dense rows.
template <typename VecT, typename OffT, typename E>
__global__ void __launch_bounds__(kThreads)
    jagged_dense_add_kernel(JaggedDev s, const VecT* __restrict__ x_values,
                            const VecT* __restrict__ y, VecT* __restrict__ out,
                            int64_t num_dense_rows, uint32_t vecs_per_row, int rows_per_cta) {
  __shared__ int64_t pair_row[kMaxRowsPerCta];
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * rows_per_cta;
  const int64_t left = num_dense_rows - row0;
  const int nrows = left < rows_per_cta ? static_cast<int>(left) : rows_per_cta;
  for (int t = threadIdx.x; t < nrows; t += kThreads) pair_row[t] = jagged_row_of<OffT>(s, row0 + t);
  __syncthreads();

  const uint32_t nvec = static_cast<uint32_t>(nrows) * vecs_per_row;
  const int64_t dense_base = row0 * vecs_per_row;
  for (uint32_t i0 = threadIdx.x; i0 < nvec; i0 += kThreads * kUnroll) {
    VecT xv[kUnroll], yv[kUnroll];
    bool has_x[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = i0 + u * kThreads;
      has_x[u] = false;
      if (i < nvec) {
        const uint32_t r = i / vecs_per_row;
        const uint32_t c = i - r * vecs_per_row;
        const int64_t pr = pair_row[r];
        yv[u] = load_stream(y + dense_base + i);
        if (pr >= 0) {
          xv[u] = load_stream(x_values + pr * vecs_per_row + c);
          has_x[u] = true;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = i0 + u * kThreads;
      if (i < nvec) {
        // y + 0 is written as an add too, so that -0.0 + 0.0 gives what the dense add gives.
        const VecT xx = has_x[u] ? xv[u] : zero_vec<VecT>();
        store_stream(out + dense_base + i, add_elems<E, VecT>(xx, yv[u]));
      }
    }
  }
}

// One jagged dimension, iterating over rows of values: row r belongs to the bag b with
// offsets[b] <= r < offsets[b+1] (binary search), position l = r - offsets[b]; it takes
// dense[b, l] when l < max_length and zeros otherwise. Work is proportional to the jagged size,
// not to the padded size.
template <typename VecT, typename OffT>
__global__ void __launch_bounds__(kThreads)
    dense_to_jagged_1d_kernel(const OffT* __restrict__ offsets, int64_t outer_size,
                              int64_t max_length, const VecT* __restrict__ dense,
                              VecT* __restrict__ values, int64_t total_rows, uint32_t vecs_per_row,
                              int rows_per_cta) {
  __shared__ int64_t pair_row[kMaxRowsPerCta];
  const int64_t row0 = static_cast<int64_t>(blockIdx.x) * rows_per_cta;
  const int64_t left = total_rows - row0;
  const int nrows = left < rows_per_cta ? static_cast<int>(left) : rows_per_cta;
  for (int t = threadIdx.x; t < nrows; t += kThreads) {
    const int64_t r = row0 + t;
    // first j in [0, outer_size] with offsets[j] > r
    int64_t lo = 0, hi = outer_size + 1;
    while (lo < hi) {
      const int64_t mid = (lo + hi) >> 1;
      if (static_cast<int64_t>(__ldg(offsets + mid)) > r) {
        hi = mid;
      } else {
        lo = mid + 1;
      }
    }
    int64_t pr = -1;
    if (lo >= 1 && lo <= outer_size) {
      const int64_t b = lo - 1;
      const int64_t l = r - static_cast<int64_t>(__ldg(offsets + b));
      if (l < max_length) pr = b * max_length + l;
    }
    pair_row[t] = pr;
  }
  __syncthreads();

  const uint32_t nvec = static_cast<uint32_t>(nrows) * vecs_per_row;
  const int64_t base = row0 * vecs_per_row;
  for (uint32_t i0 = threadIdx.x; i0 < nvec; i0 += kThreads * kUnroll) {
    VecT v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = i0 + u * kThreads;
      if (i < nvec) {
        const uint32_t r = i / vecs_per_row;
        const uint32_t c = i - r * vecs_per_row;
        const int64_t pr = pair_row[r];
        v[u] = pr >= 0 ? load_stream(dense + pr * vecs_per_row + c) : zero_vec<VecT>();
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = i0 + u * kThreads;
      if (i < nvec) store_stream(values + base + i, v[u]);
    }
  }
}

struct Plan {
  JaggedDev dev;
  int64_t num_dense_rows;
  int64_t row_bytes;
  int vec_bytes;
  uint32_t vecs_per_row;
  int rows_per_cta;
};

int make_plan(const b200tbe_jagged_shape* s, const void* a, const void* b, const void* c,
              Plan* plan) {
  if (s == nullptr) return B200TBE_ERR_BAD_ARG;
  if (s->num_jagged_dims < 1 || s->num_jagged_dims > B200TBE_MAX_JAGGED_DIMS)
    return B200TBE_ERR_UNSUPPORTED;
  if (s->offset_bytes != 4 && s->offset_bytes != 8) return B200TBE_ERR_BAD_ARG;
  if (s->elem_bytes != 1 && s->elem_bytes != 2 && s->elem_bytes != 4 && s->elem_bytes != 8)
    return B200TBE_ERR_UNSUPPORTED;
  if (s->outer_size < 0 || s->inner_size < 0 || s->total_rows < 0) return B200TBE_ERR_BAD_ARG;
  plan->dev.n = s->num_jagged_dims;
  plan->dev.total_rows = s->total_rows;
  int64_t rows = s->outer_size;
  for (int d = 0; d < B200TBE_MAX_JAGGED_DIMS; ++d) {
    plan->dev.offsets[d] = nullptr;
    plan->dev.max_lengths[d] = 1;
  }
  for (int d = 0; d < s->num_jagged_dims; ++d) {
    if (s->max_lengths[d] < 0) return B200TBE_ERR_BAD_ARG;
    if (s->offsets[d] == nullptr) return B200TBE_ERR_BAD_ARG;
    plan->dev.offsets[d] = s->offsets[d];
    plan->dev.max_lengths[d] = s->max_lengths[d];
    rows *= s->max_lengths[d];
  }
  plan->num_dense_rows = rows;
  plan->row_bytes = s->inner_size * s->elem_bytes;
  int vb = 16;
  while (vb > s->elem_bytes &&
         (plan->row_bytes % vb != 0 || !aligned_to(a, vb) || !aligned_to(b, vb) ||
          !aligned_to(c, vb)))
    vb >>= 1;
  plan->vec_bytes = vb;
  const int64_t vpr = plan->row_bytes / vb;
  if (vpr > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  plan->vecs_per_row = static_cast<uint32_t>(vpr);
  int64_t rpc = vpr > 0 ? kTileVecs / vpr : 1;
  if (rpc < 1) rpc = 1;
  if (rpc > kMaxRowsPerCta) rpc = kMaxRowsPerCta;
  plan->rows_per_cta = static_cast<int>(rpc);
  return B200TBE_OK;
}

inline int64_t num_ctas(int64_t rows, int rows_per_cta) {
  return (rows + rows_per_cta - 1) / rows_per_cta;
}

template <typename VecT>
VecT make_pad(uint64_t pad_bits, int elem_bytes) {
  unsigned char bytes[16];
  for (int i = 0; i < 16; ++i) bytes[i] = static_cast<unsigned char>(pad_bits >> (8 * (i % elem_bytes)));
  VecT v;
  memcpy(&v, bytes, sizeof(VecT));
  return v;
}

template <typename VecT, typename OffT, int kMode>
int launch_rows(const Plan& pl, const void* src, void* dst, uint64_t pad_bits, int elem_bytes,
                cudaStream_t stream) {
  const int64_t ctas = num_ctas(pl.num_dense_rows, pl.rows_per_cta);
  if (ctas > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  jagged_dense_rows_kernel<VecT, OffT, kMode>
      <<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(
          pl.dev, static_cast<const VecT*>(src), static_cast<VecT*>(dst),
          make_pad<VecT>(pad_bits, elem_bytes), pl.num_dense_rows, pl.vecs_per_row,
          pl.rows_per_cta);
  return launch_status();
}

template <typename OffT, int kMode>
int dispatch_rows(const Plan& pl, const void* src, void* dst, uint64_t pad_bits, int elem_bytes,
                  cudaStream_t stream) {
  switch (pl.vec_bytes) {
    case 16: return launch_rows<uint4, OffT, kMode>(pl, src, dst, pad_bits, elem_bytes, stream);
    case 8: return launch_rows<unsigned long long, OffT, kMode>(pl, src, dst, pad_bits, elem_bytes, stream);
    case 4: return launch_rows<uint32_t, OffT, kMode>(pl, src, dst, pad_bits, elem_bytes, stream);
    case 2: return launch_rows<uint16_t, OffT, kMode>(pl, src, dst, pad_bits, elem_bytes, stream);
    default: return launch_rows<uint8_t, OffT, kMode>(pl, src, dst, pad_bits, elem_bytes, stream);
  }
}

template <typename VecT, typename OffT>
int launch_d2j_1d(const Plan& pl, const b200tbe_jagged_shape* s, const void* dense, void* values,
                  cudaStream_t stream) {
  const int64_t ctas = num_ctas(s->total_rows, pl.rows_per_cta);
  if (ctas > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  dense_to_jagged_1d_kernel<VecT, OffT><<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(
      static_cast<const OffT*>(s->offsets[0]), s->outer_size, s->max_lengths[0],
      static_cast<const VecT*>(dense), static_cast<VecT*>(values), s->total_rows, pl.vecs_per_row,
      pl.rows_per_cta);
  return launch_status();
}

template <typename OffT>
int dispatch_d2j_1d(const Plan& pl, const b200tbe_jagged_shape* s, const void* dense, void* values,
                    cudaStream_t stream) {
  switch (pl.vec_bytes) {
    case 16: return launch_d2j_1d<uint4, OffT>(pl, s, dense, values, stream);
    case 8: return launch_d2j_1d<unsigned long long, OffT>(pl, s, dense, values, stream);
    case 4: return launch_d2j_1d<uint32_t, OffT>(pl, s, dense, values, stream);
    case 2: return launch_d2j_1d<uint16_t, OffT>(pl, s, dense, values, stream);
    default: return launch_d2j_1d<uint8_t, OffT>(pl, s, dense, values, stream);
  }
}

template <typename VecT, typename OffT, typename E>
int launch_add(const Plan& pl, const void* x, const void* y, void* out, cudaStream_t stream) {
  const int64_t ctas = num_ctas(pl.num_dense_rows, pl.rows_per_cta);
  if (ctas > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  jagged_dense_add_kernel<VecT, OffT, E><<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(
      pl.dev, static_cast<const VecT*>(x), static_cast<const VecT*>(y), static_cast<VecT*>(out),
      pl.num_dense_rows, pl.vecs_per_row, pl.rows_per_cta);
  return launch_status();
}

template <typename OffT, typename E>
int dispatch_add(const Plan& pl, const void* x, const void* y, void* out, cudaStream_t stream) {
  switch (pl.vec_bytes) {
    case 16: return launch_add<uint4, OffT, E>(pl, x, y, out, stream);
    case 8: return launch_add<unsigned long long, OffT, E>(pl, x, y, out, stream);
    case 4:
      if (sizeof(E) <= 4) return launch_add<uint32_t, OffT, E>(pl, x, y, out, stream);
      return B200TBE_ERR_UNSUPPORTED;
    default: break;
  }
  return B200TBE_ERR_UNSUPPORTED;
}

// 2-byte vectors only exist for 2-byte element types.
template <typename OffT, typename E>
int dispatch_add16(const Plan& pl, const void* x, const void* y, void* out, cudaStream_t stream) {
  if (pl.vec_bytes == 2) return launch_add<uint16_t, OffT, E>(pl, x, y, out, stream);
  return dispatch_add<OffT, E>(pl, x, y, out, stream);
}

}  // namespace
}  // namespace b200tbe

using namespace b200tbe;

extern "C" int b200tbe_jagged_to_padded_dense(const b200tbe_jagged_shape* s, const void* values,
                                              void* dense, uint64_t pad_bits,
                                              b200tbe_stream_t stream_) {
  Plan pl;
  const int st = make_plan(s, values, dense, nullptr, &pl);
  if (st != B200TBE_OK) return st;
  if (pl.num_dense_rows == 0 || pl.row_bytes == 0) return B200TBE_OK;
  if (dense == nullptr || (values == nullptr && s->total_rows > 0)) return B200TBE_ERR_BAD_ARG;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (s->offset_bytes == 8)
    return dispatch_rows<int64_t, kToDense>(pl, values, dense, pad_bits, s->elem_bytes, stream);
  return dispatch_rows<int32_t, kToDense>(pl, values, dense, pad_bits, s->elem_bytes, stream);
}

extern "C" int b200tbe_dense_to_jagged(const b200tbe_jagged_shape* s, const void* dense,
                                       void* values, b200tbe_stream_t stream_) {
  Plan pl;
  const int st = make_plan(s, dense, values, nullptr, &pl);
  if (st != B200TBE_OK) return st;
  if (s->total_rows == 0 || pl.row_bytes == 0) return B200TBE_OK;
  if (values == nullptr || (dense == nullptr && pl.num_dense_rows > 0)) return B200TBE_ERR_BAD_ARG;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (s->num_jagged_dims == 1) {
    if (s->offset_bytes == 8) return dispatch_d2j_1d<int64_t>(pl, s, dense, values, stream);
    return dispatch_d2j_1d<int32_t>(pl, s, dense, values, stream);
  }
  // Nested offsets: rows that the padded shape cannot reach stay zero.
  if (cudaMemsetAsync(values, 0, static_cast<size_t>(s->total_rows) * pl.row_bytes, stream) !=
      cudaSuccess)
    return B200TBE_ERR_LAUNCH;
  if (pl.num_dense_rows == 0) return B200TBE_OK;
  if (s->offset_bytes == 8)
    return dispatch_rows<int64_t, kFromDense>(pl, dense, values, 0, s->elem_bytes, stream);
  return dispatch_rows<int32_t, kFromDense>(pl, dense, values, 0, s->elem_bytes, stream);
}

extern "C" int b200tbe_jagged_dense_elementwise_add(const b200tbe_jagged_shape* s,
                                                    const void* x_values, const void* y, void* out,
                                                    b200tbe_stream_t stream_) {
  Plan pl;
  const int st = make_plan(s, x_values, y, out, &pl);
  if (st != B200TBE_OK) return st;
  if (pl.num_dense_rows == 0 || pl.row_bytes == 0) return B200TBE_OK;
  if (y == nullptr || out == nullptr || (x_values == nullptr && s->total_rows > 0))
    return B200TBE_ERR_BAD_ARG;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const bool o64 = s->offset_bytes == 8;
  switch (s->dtype) {
    case B200TBE_FP32:
      if (s->elem_bytes != 4) return B200TBE_ERR_BAD_ARG;
      return o64 ? dispatch_add<int64_t, float>(pl, x_values, y, out, stream)
                 : dispatch_add<int32_t, float>(pl, x_values, y, out, stream);
    case B200TBE_FP16:
      if (s->elem_bytes != 2) return B200TBE_ERR_BAD_ARG;
      return o64 ? dispatch_add16<int64_t, __half>(pl, x_values, y, out, stream)
                 : dispatch_add16<int32_t, __half>(pl, x_values, y, out, stream);
    case B200TBE_BF16:
      if (s->elem_bytes != 2) return B200TBE_ERR_BAD_ARG;
      return o64 ? dispatch_add16<int64_t, __nv_bfloat16>(pl, x_values, y, out, stream)
                 : dispatch_add16<int32_t, __nv_bfloat16>(pl, x_values, y, out, stream);
    default:
      return B200TBE_ERR_UNSUPPORTED;
  }
}
