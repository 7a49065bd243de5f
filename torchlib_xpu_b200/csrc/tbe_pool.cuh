// Warp-level pieces shared by the TBE forward kernels: typed row vectors, pooled-value stores and
// the gather loop over rows made of whole 16-byte vectors.
#pragma once

#include "common.cuh"

namespace b200tbe {

template <typename WT>
struct RowVec;
template <>
struct RowVec<float> {
  static constexpr int kElems = 4;
  static __device__ __forceinline__ void fma(float* acc, uint4 v, float w) {
    acc[0] = fmaf(__uint_as_float(v.x), w, acc[0]);
    acc[1] = fmaf(__uint_as_float(v.y), w, acc[1]);
    acc[2] = fmaf(__uint_as_float(v.z), w, acc[2]);
    acc[3] = fmaf(__uint_as_float(v.w), w, acc[3]);
  }
  static __device__ __forceinline__ void add(float* acc, uint4 v) {
    acc[0] += __uint_as_float(v.x);
    acc[1] += __uint_as_float(v.y);
    acc[2] += __uint_as_float(v.z);
    acc[3] += __uint_as_float(v.w);
  }
  static __device__ __forceinline__ float scalar(const char* p) {
    return __ldg(reinterpret_cast<const float*>(p));
  }
};
template <>
struct RowVec<__half> {
  static constexpr int kElems = 8;
  static __device__ __forceinline__ void fma(float* acc, uint4 v, float w) {
    const float2 a = half2_bits_to_float2(v.x), b = half2_bits_to_float2(v.y),
                 c = half2_bits_to_float2(v.z), d = half2_bits_to_float2(v.w);
    acc[0] = fmaf(a.x, w, acc[0]);
    acc[1] = fmaf(a.y, w, acc[1]);
    acc[2] = fmaf(b.x, w, acc[2]);
    acc[3] = fmaf(b.y, w, acc[3]);
    acc[4] = fmaf(c.x, w, acc[4]);
    acc[5] = fmaf(c.y, w, acc[5]);
    acc[6] = fmaf(d.x, w, acc[6]);
    acc[7] = fmaf(d.y, w, acc[7]);
  }
  static __device__ __forceinline__ void add(float* acc, uint4 v) {
    const float2 a = half2_bits_to_float2(v.x), b = half2_bits_to_float2(v.y),
                 c = half2_bits_to_float2(v.z), d = half2_bits_to_float2(v.w);
    acc[0] += a.x;
    acc[1] += a.y;
    acc[2] += b.x;
    acc[3] += b.y;
    acc[4] += c.x;
    acc[5] += c.y;
    acc[6] += d.x;
    acc[7] += d.y;
  }
  static __device__ __forceinline__ float scalar(const char* p) {
    return __half2float(__ldg(reinterpret_cast<const __half*>(p)));
  }
};

// Writes n (4 or 8) consecutive pooled values with the widest store the address allows.
template <typename OT, int kN>
__device__ __forceinline__ void store_pooled(OT* p, const float* v);

template <>
__device__ __forceinline__ void store_pooled<float, 4>(float* p, const float* v) {
  if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = v[i];
  }
}
template <>
__device__ __forceinline__ void store_pooled<float, 8>(float* p, const float* v) {
  store_pooled<float, 4>(p, v);
  store_pooled<float, 4>(p + 4, v + 4);
}
template <>
__device__ __forceinline__ void store_pooled<__half, 4>(__half* p, const float* v) {
  if ((reinterpret_cast<uintptr_t>(p) & 7) == 0) {
    *reinterpret_cast<uint2*>(p) =
        make_uint2(float2_to_half2_bits(v[0], v[1]), float2_to_half2_bits(v[2], v[3]));
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __float2half_rn(v[i]);
  }
}
template <>
__device__ __forceinline__ void store_pooled<__half, 8>(__half* p, const float* v) {
  if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    *reinterpret_cast<uint4*>(p) =
        make_uint4(float2_to_half2_bits(v[0], v[1]), float2_to_half2_bits(v[2], v[3]),
                   float2_to_half2_bits(v[4], v[5]), float2_to_half2_bits(v[6], v[7]));
  } else {
    store_pooled<__half, 4>(p, v);
    store_pooled<__half, 4>(p + 4, v + 4);
  }
}

__device__ __forceinline__ float to_out(float v, float*) { return v; }
__device__ __forceinline__ __half to_out(float v, __half*) { return __float2half_rn(v); }


// Run of n pooled values (n a multiple of 4) starting at p.
template <typename OT>
__device__ __forceinline__ void store_pooled_run(OT* p, const float* v, int n) {
#pragma unroll 1
  for (int i = 0; i + 8 <= n; i += 8) store_pooled<OT, 8>(p + i, v + i);
  if (n & 4) store_pooled<OT, 4>(p + (n & ~7), v + (n & ~7));
}

// One bag's lookups [start, end) over a table whose rows are row_vecs whole 16-byte vectors,
// row_stride bytes apart. The warp splits into 32/gs groups of gs lanes; each group accumulates a
// different subset of the bag's rows into acc, and the caller combines the groups afterwards.
// Indices out of [0, num_rows) are skipped and flagged when num_rows >= 0.
template <typename WT, typename IndexT, int kVPL, int kUnroll>
__device__ __forceinline__ void pool_vector_rows(float (&acc)[kVPL][RowVec<WT>::kElems],
                                                 const char* table, int64_t row_stride,
                                                 int row_vecs, int gs, const void* indices,
                                                 const float* per_sample_weights, int64_t start,
                                                 int64_t end, int64_t num_rows, int32_t* status,
                                                 int lane) {
  const int rows_per_step = 32 / gs;
  const int g = lane / gs;
  const int v = lane - g * gs;
  const bool weighted = per_sample_weights != nullptr;
  for (int64_t c = start; c < end; c += 32) {
    const int n = end - c < 32 ? static_cast<int>(end - c) : 32;
    int64_t my_idx = -1;
    float my_w = 1.f;
    if (lane < n) {
      my_idx = load_index<IndexT>(indices, c + lane);
      if (weighted) my_w = __ldg(per_sample_weights + c + lane);
      if (num_rows >= 0 && (my_idx < 0 || my_idx >= num_rows)) {
        atomicOr(status, B200TBE_DEV_INDEX_OUT_OF_RANGE);
        my_idx = -1;
      }
    }
    for (int j = 0; j < n; j += rows_per_step * kUnroll) {
      uint4 buf[kUnroll][kVPL];
      float w[kUnroll];
      bool ok[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int rr = j + u * rows_per_step + g;
        const int64_t idx = __shfl_sync(kFullMask, my_idx, rr & 31);
        w[u] = __shfl_sync(kFullMask, my_w, rr & 31);
        ok[u] = rr < n && idx >= 0;
        if (ok[u]) {
          const char* row = table + idx * row_stride;
#pragma unroll
          for (int k = 0; k < kVPL; ++k) {
            const int vv = k * 32 + v;
            if (vv < row_vecs) buf[u][k] = ldg_stream16(row + (static_cast<int64_t>(vv) << 4));
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (ok[u]) {
#pragma unroll
          for (int k = 0; k < kVPL; ++k) {
            if (k * 32 + v < row_vecs) {
              if (weighted) {
                RowVec<WT>::fma(acc[k], buf[u][k], w[u]);
              } else {
                RowVec<WT>::add(acc[k], buf[u][k]);
              }
            }
          }
        }
      }
    }
  }
}

// Lanes per row for rows of row_vecs 16-byte vectors: row_vecs rounded up to a power of two, 32 at
// most.
__device__ __forceinline__ int lanes_per_row(int row_vecs) {
  int gs = 32;
  while (gs > 1 && (gs >> 1) >= row_vecs) gs >>= 1;
  return gs;
}

}  // namespace b200tbe
