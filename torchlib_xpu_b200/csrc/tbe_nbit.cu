// Quantised-inference TBE forward: INT8 / INT4 (/ INT2) row-wise quantised tables with an fp16
// {scale, bias} header per row, plus FP16 / FP32 tables, mixed per table; one warp per bag.
//
// Quantised fast path. A row is a 4-byte header followed by the payload, so the payload is 4-byte
// but not 16-byte aligned. Lane c of a row's lane group takes payload bytes [16c, 16c+16): it loads
// the aligned 16 bytes at row+16c and the 4 bytes at row+16c+16 (same cache lines, second load is
// an L1/coalescer hit) and keeps words 1..3 of the first plus the extra word. That way every lane
// dequantises 16 payload bytes -- no lane idles on the header or on row padding, which matters
// because this kernel is bound by instruction issue (two int->float conversions + FMAs per payload
// byte for INT4), not only by HBM. A group is payload/16 lanes rounded up to a power of two, the
// warp handles 32/gs rows per load instruction. q*scale is accumulated per element in fp32 and the
// per-row bias is accumulated once per row and added at the end.
#include "tbe_pool.cuh"

namespace b200tbe {
namespace {

constexpr int kNbitWarps = 8;
constexpr int kNbitThreads = kNbitWarps * kWarpSize;

struct NbitDev {
  const uint8_t* dev_weights;
  const int64_t* weights_offsets;
  const uint8_t* weights_tys;
  const int32_t* D_offsets;
  const int64_t* rows_per_table;
  const void* indices;
  const void* offsets;
  const float* per_sample_weights;
  void* outputs[B200TBE_MAX_DESTS];
  int64_t output_stride;
  int64_t output_col_offset;
  int64_t rows_per_dest;
  int32_t T;
  int32_t B;
  int32_t row_alignment;
  int32_t pooling_mode;
  int32_t* status;
};

// acc[i] += s * q_i for the 16 payload bytes in w[0..3].
template <int kBits>
struct Dequant;

template <>
struct Dequant<8> {
  static constexpr int kElems = 16;  // per 16 payload bytes
  static __device__ __forceinline__ void accumulate(float2* acc, const uint32_t (&w)[4], float s) {
    const float2 ss = make_float2(s, s);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 lo = make_float2(static_cast<float>(w[i] & 0xffu),
                                    static_cast<float>((w[i] >> 8) & 0xffu));
      const float2 hi = make_float2(static_cast<float>((w[i] >> 16) & 0xffu),
                                    static_cast<float>(w[i] >> 24));
      acc[2 * i] = __ffma2_rn(lo, ss, acc[2 * i]);
      acc[2 * i + 1] = __ffma2_rn(hi, ss, acc[2 * i + 1]);
    }
  }
};

template <>
struct Dequant<4> {
  static constexpr int kElems = 32;
  static __device__ __forceinline__ void accumulate(float2* acc, const uint32_t (&w)[4], float s) {
    const float2 ss = make_float2(s, s);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 q = make_float2(static_cast<float>((w[i] >> (8 * k)) & 0xfu),
                                     static_cast<float>((w[i] >> (8 * k + 4)) & 0xfu));
        acc[4 * i + k] = __ffma2_rn(q, ss, acc[4 * i + k]);
      }
    }
  }
};

__device__ __forceinline__ float2 header_scale_bias(uint32_t header) {
  return half2_bits_to_float2(header);
}

// Quantised rows whose payload is chunks whole 16-byte pieces (chunks <= 32) and whose stride and
// base are 16-byte aligned. Pools one bag and writes the result.
template <int kBits, typename OT, typename IndexT>
__device__ __forceinline__ void pool_quantised_bag(const NbitDev& p, const uint8_t* table,
                                                   int64_t row_stride, int chunks, int64_t start,
                                                   int64_t end, int64_t num_rows, OT* out,
                                                   int lane) {
  constexpr int kE = Dequant<kBits>::kElems;
  constexpr int kUnroll = 2;
  const int gs = lanes_per_row(chunks);
  const int rows_per_step = 32 / gs;
  const int g = lane / gs;
  const int c = lane - g * gs;
  const bool weighted = p.per_sample_weights != nullptr;

  float2 acc[kE / 2];
#pragma unroll
  for (int e = 0; e < kE / 2; ++e) acc[e] = make_float2(0.f, 0.f);
  float bias_sum = 0.f;

  for (int64_t pos = start; pos < end; pos += 32) {
    const int n = end - pos < 32 ? static_cast<int>(end - pos) : 32;
    int64_t my_idx = -1;
    float my_w = 1.f;
    if (lane < n) {
      my_idx = load_index<IndexT>(p.indices, pos + lane);
      if (weighted) my_w = __ldg(p.per_sample_weights + pos + lane);
      if (num_rows >= 0 && (my_idx < 0 || my_idx >= num_rows)) {
        atomicOr(p.status, B200TBE_DEV_INDEX_OUT_OF_RANGE);
        my_idx = -1;
      }
    }
    for (int j = 0; j < n; j += rows_per_step * kUnroll) {
      uint4 a[kUnroll];
      uint32_t extra[kUnroll];
      float w[kUnroll];
      bool ok[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int rr = j + u * rows_per_step + g;
        const int64_t idx = __shfl_sync(kFullMask, my_idx, rr & 31);
        w[u] = __shfl_sync(kFullMask, my_w, rr & 31);
        ok[u] = rr < n && idx >= 0 && c < chunks;
        a[u] = make_uint4(0, 0, 0, 0);
        extra[u] = 0;
        if (ok[u]) {
          const uint8_t* src = table + idx * row_stride + (c << 4);
          a[u] = ldg_stream16(src);
          extra[u] = ldg_stream4(src + 16);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        // the header sits in word 0 of the group's first lane
        const uint32_t header = __shfl_sync(kFullMask, a[u].x, g * gs);
        if (ok[u]) {
          const float2 sb = header_scale_bias(header);
          const uint32_t words[4] = {a[u].y, a[u].z, a[u].w, extra[u]};
          Dequant<kBits>::accumulate(acc, words, sb.x * w[u]);
          bias_sum = fmaf(sb.y, w[u], bias_sum);
        }
      }
    }
  }
  for (int o = 16; o >= gs; o >>= 1) {
#pragma unroll
    for (int e = 0; e < kE / 2; ++e) {
      acc[e].x += __shfl_xor_sync(kFullMask, acc[e].x, o);
      acc[e].y += __shfl_xor_sync(kFullMask, acc[e].y, o);
    }
    bias_sum += __shfl_xor_sync(kFullMask, bias_sum, o);
  }
  float scale = 1.f;
  if (p.pooling_mode == B200TBE_POOL_MEAN && end > start) scale = 1.f / static_cast<float>(end - start);
  if (g == 0 && c < chunks) {
    OT* dst = out + c * kE;
#pragma unroll
    for (int e = 0; e < kE; e += 8) {
      float r[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        r[2 * i] = (acc[e / 2 + i].x + bias_sum) * scale;
        r[2 * i + 1] = (acc[e / 2 + i].y + bias_sum) * scale;
      }
      store_pooled<OT, 8>(dst + e, r);
    }
  }
}

// Any table type, any D, any alignment: 128 output columns at a time, element (col0 + i*32 + lane)
// in accumulator i, one byte-sized load per element. Correct everywhere, fast nowhere.
template <typename OT, typename IndexT>
__device__ __noinline__ void pool_bag_generic(const void* indices, const float* per_sample_weights,
                                              int pooling_mode, int32_t* status, int ty,
                                              const uint8_t* table, int64_t row_stride, int D,
                                              int64_t start, int64_t end, int64_t num_rows, OT* out,
                                              int lane) {
  const bool weighted = per_sample_weights != nullptr;
  float scale = 1.f;
  if (pooling_mode == B200TBE_POOL_MEAN && end > start) scale = 1.f / static_cast<float>(end - start);
  for (int col0 = 0; col0 < D; col0 += 128) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int64_t pos = start; pos < end; ++pos) {
      const int64_t idx = load_index<IndexT>(indices, pos);
      const float w = weighted ? __ldg(per_sample_weights + pos) : 1.f;
      if (num_rows >= 0 && (idx < 0 || idx >= num_rows)) {
        if (lane == 0 && col0 == 0) atomicOr(status, B200TBE_DEV_INDEX_OUT_OF_RANGE);
        continue;
      }
      const uint8_t* row = table + idx * row_stride;
      float s = 1.f, bsh = 0.f;
      if (ty == B200TBE_INT8 || ty == B200TBE_INT4 || ty == B200TBE_INT2) {
        const unsigned lo = __ldg(reinterpret_cast<const unsigned short*>(row));
        const unsigned hi = __ldg(reinterpret_cast<const unsigned short*>(row) + 1);
        const float2 sb = header_scale_bias(lo | (hi << 16));
        s = sb.x;
        bsh = sb.y;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int e = col0 + i * 32 + lane;
        if (e < D) {
          float val;
          if (ty == B200TBE_INT8) {
            val = fmaf(static_cast<float>(__ldg(row + 4 + e)), s, bsh);
          } else if (ty == B200TBE_INT4) {
            const unsigned byte = __ldg(row + 4 + (e >> 1));
            val = fmaf(static_cast<float>((byte >> ((e & 1) * 4)) & 0xfu), s, bsh);
          } else if (ty == B200TBE_INT2) {
            const unsigned byte = __ldg(row + 4 + (e >> 2));
            val = fmaf(static_cast<float>((byte >> ((e & 3) * 2)) & 0x3u), s, bsh);
          } else if (ty == B200TBE_FP16) {
            val = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(row) + e)));
          } else {
            val = __ldg(reinterpret_cast<const float*>(row) + e);
          }
          acc[i] = fmaf(val, w, acc[i]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = col0 + i * 32 + lane;
      if (e < D) out[e] = to_out(acc[i] * scale, static_cast<OT*>(nullptr));
    }
  }
}

// FP16 / FP32 tables inside the quantised op: rows of whole 16-byte vectors, at most 32 of them.
template <typename WT, typename OT, typename IndexT>
__device__ __forceinline__ void pool_float_bag(const NbitDev& p, const uint8_t* table,
                                               int64_t row_stride, int row_vecs, int64_t start,
                                               int64_t end, int64_t num_rows, OT* out, int lane) {
  constexpr int kE = RowVec<WT>::kElems;
  float acc[1][kE];
#pragma unroll
  for (int e = 0; e < kE; ++e) acc[0][e] = 0.f;
  const int gs = lanes_per_row(row_vecs);
  const int g = lane / gs;
  const int v = lane - g * gs;
  pool_vector_rows<WT, IndexT, 1, 2>(acc, reinterpret_cast<const char*>(table), row_stride,
                                     row_vecs, gs, p.indices, p.per_sample_weights, start, end,
                                     num_rows, p.status, lane);
  for (int o = 16; o >= gs; o >>= 1) {
#pragma unroll
    for (int e = 0; e < kE; ++e) acc[0][e] += __shfl_xor_sync(kFullMask, acc[0][e], o);
  }
  float scale = 1.f;
  if (p.pooling_mode == B200TBE_POOL_MEAN && end > start) scale = 1.f / static_cast<float>(end - start);
  if (g == 0 && v < row_vecs) {
#pragma unroll
    for (int e = 0; e < kE; ++e) acc[0][e] *= scale;
    store_pooled<OT, kE>(out + v * kE, acc[0]);
  }
}

__device__ __forceinline__ int64_t round_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

template <typename OT, typename IndexT>
__global__ void __launch_bounds__(kNbitThreads) tbe_nbit_forward_kernel(NbitDev p) {
  const int lane = threadIdx.x & 31;
  const int64_t bag = static_cast<int64_t>(blockIdx.x) * kNbitWarps + (threadIdx.x >> 5);
  if (bag >= static_cast<int64_t>(p.T) * p.B) return;
  const int t = static_cast<int>(bag / p.B);
  const int b = static_cast<int>(bag - static_cast<int64_t>(t) * p.B);

  const int ty = __ldg(p.weights_tys + t);
  const int D_begin = __ldg(p.D_offsets + t);
  const int D = __ldg(p.D_offsets + t + 1) - D_begin;
  const uint8_t* table = p.dev_weights + __ldg(p.weights_offsets + t);
  const int64_t num_rows = p.rows_per_table ? __ldg(p.rows_per_table + t) : -1;
  const int64_t start = load_index<IndexT>(p.offsets, bag);
  const int64_t end = load_index<IndexT>(p.offsets, bag + 1);

  const int dest = static_cast<int>(b / p.rows_per_dest);
  const int64_t dest_row = b - dest * p.rows_per_dest;
  OT* out = static_cast<OT*>(p.outputs[dest]) + dest_row * p.output_stride + p.output_col_offset +
            D_begin;

  int64_t payload;  // bytes
  int header = 4;
  switch (ty) {
    case B200TBE_INT8: payload = D; break;
    case B200TBE_INT4: payload = (D + 1) / 2; break;
    case B200TBE_INT2: payload = (D + 3) / 4; break;
    case B200TBE_FP16: payload = int64_t{D} * 2; header = 0; break;
    default: payload = int64_t{D} * 4; header = 0; break;
  }
  const int64_t row_stride = round_up(header + payload, p.row_alignment);
  const bool aligned16 = (row_stride & 15) == 0 && (reinterpret_cast<uintptr_t>(table) & 15) == 0 &&
                         (payload & 15) == 0 && payload <= 512;
  if (aligned16 && ty == B200TBE_INT8) {
    pool_quantised_bag<8, OT, IndexT>(p, table, row_stride, static_cast<int>(payload >> 4), start,
                                      end, num_rows, out, lane);
  } else if (aligned16 && ty == B200TBE_INT4 && (D & 1) == 0) {
    pool_quantised_bag<4, OT, IndexT>(p, table, row_stride, static_cast<int>(payload >> 4), start,
                                      end, num_rows, out, lane);
  } else if (aligned16 && ty == B200TBE_FP16) {
    pool_float_bag<__half, OT, IndexT>(p, table, row_stride, static_cast<int>(payload >> 4), start,
                                       end, num_rows, out, lane);
  } else if (aligned16 && ty == B200TBE_FP32) {
    pool_float_bag<float, OT, IndexT>(p, table, row_stride, static_cast<int>(payload >> 4), start,
                                      end, num_rows, out, lane);
  } else {
    pool_bag_generic<OT, IndexT>(p.indices, p.per_sample_weights, p.pooling_mode, p.status, ty, table, row_stride, D, start, end, num_rows, out, lane);
  }
}

template <typename OT, typename IndexT>
int launch_nbit(const NbitDev& d, cudaStream_t stream) {
  const int64_t bags = static_cast<int64_t>(d.T) * d.B;
  const int64_t ctas = (bags + kNbitWarps - 1) / kNbitWarps;
  if (ctas > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  tbe_nbit_forward_kernel<OT, IndexT><<<static_cast<unsigned>(ctas), kNbitThreads, 0, stream>>>(d);
  return launch_status();
}

}  // namespace
}  // namespace b200tbe

using namespace b200tbe;

extern "C" int b200tbe_nbit_forward(const b200tbe_nbit_forward_params* p,
                                    b200tbe_stream_t stream_) {
  if (p == nullptr) return B200TBE_ERR_BAD_ARG;
  if (p->T < 0 || p->B < 0 || p->max_D < 0) return B200TBE_ERR_BAD_ARG;
  if (p->T == 0 || p->B == 0) return B200TBE_OK;
  if (p->dev_weights == nullptr || p->weights_offsets == nullptr || p->weights_tys == nullptr ||
      p->D_offsets == nullptr || p->offsets == nullptr)
    return B200TBE_ERR_BAD_ARG;
  if (p->index_bytes != 4 && p->index_bytes != 8) return B200TBE_ERR_BAD_ARG;
  if (p->row_alignment < 1) return B200TBE_ERR_BAD_ARG;
  if (p->num_dests < 1 || p->num_dests > B200TBE_MAX_DESTS) return B200TBE_ERR_BAD_ARG;
  if (p->rows_per_dest < 1 || p->rows_per_dest * p->num_dests < p->B) return B200TBE_ERR_BAD_ARG;
  if (p->rows_per_table != nullptr && p->status == nullptr) return B200TBE_ERR_BAD_ARG;
  if (p->pooling_mode != B200TBE_POOL_SUM && p->pooling_mode != B200TBE_POOL_MEAN)
    return B200TBE_ERR_UNSUPPORTED;
  NbitDev d;
  d.dev_weights = p->dev_weights;
  d.weights_offsets = p->weights_offsets;
  d.weights_tys = p->weights_tys;
  d.D_offsets = p->D_offsets;
  d.rows_per_table = p->rows_per_table;
  d.indices = p->indices;
  d.offsets = p->offsets;
  d.per_sample_weights = p->per_sample_weights;
  for (int i = 0; i < B200TBE_MAX_DESTS; ++i) {
    d.outputs[i] = i < p->num_dests ? p->outputs[i] : nullptr;
    if (i < p->num_dests && p->outputs[i] == nullptr) return B200TBE_ERR_BAD_ARG;
  }
  d.output_stride = p->output_stride;
  d.output_col_offset = p->output_col_offset;
  d.rows_per_dest = p->rows_per_dest;
  d.T = p->T;
  d.B = p->B;
  d.row_alignment = p->row_alignment;
  d.pooling_mode = p->pooling_mode;
  d.status = p->status;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const bool i64 = p->index_bytes == 8;
  if (p->output_dtype == B200TBE_FP32)
    return i64 ? launch_nbit<float, int64_t>(d, stream) : launch_nbit<float, int32_t>(d, stream);
  if (p->output_dtype == B200TBE_FP16)
    return i64 ? launch_nbit<__half, int64_t>(d, stream) : launch_nbit<__half, int32_t>(d, stream);
  return B200TBE_ERR_UNSUPPORTED;
}
