// TBE pooled forward over fp32 / fp16 tables: one warp per bag.
//
// A row of D elements is D*sizeof(W)/16 16-byte vectors. When that is fewer than 32 the warp splits
// into 32/gs groups of gs lanes (gs = the vector count rounded up to a power of two) and each group
// fetches a different row of the bag with the same load instruction, so every lane always issues a
// full 16-byte load: D=128 fp32 -> 32 lanes x 16 B = one 512-byte row per instruction, D=128 fp16
// -> two 256-byte rows per instruction. The bag's indices are fetched 32 at a time with one
// coalesced load and handed out by shuffle. kUnroll row loads are issued back to back before any
// of them is consumed, which is what keeps enough bytes in flight to cover HBM latency. The
// accumulators are fp32 registers; groups are combined by shuffle at the end and group 0 writes the
// pooled vector. Bags are table-major, so concurrently running CTAs work on the same table and
// rows that repeat across bags (Zipf-distributed ids) are served by L2.
#include "tbe_pool.cuh"

namespace b200tbe {
namespace {

constexpr int kFwdWarps = 8;
constexpr int kFwdThreads = kFwdWarps * kWarpSize;

struct FwdDev {
  const char* dev_weights;
  const int64_t* weights_offsets;
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
  int32_t pooling_mode;
  int32_t* status;
};

// kVPL = 16-byte vectors per lane a row may need (rows of up to 32*kVPL vectors).
template <typename WT, typename OT, typename IndexT, int kVPL>
__global__ void __launch_bounds__(kFwdThreads) tbe_forward_kernel(FwdDev p) {
  constexpr int kE = RowVec<WT>::kElems;
  constexpr int kUnroll = kVPL == 1 ? 4 : (kVPL == 2 ? 2 : 1);
  const int lane = threadIdx.x & 31;
  const int64_t bag =
      static_cast<int64_t>(blockIdx.x) * kFwdWarps + (threadIdx.x >> 5);
  if (bag >= static_cast<int64_t>(p.T) * p.B) return;
  const int t = static_cast<int>(bag / p.B);
  const int b = static_cast<int>(bag - static_cast<int64_t>(t) * p.B);

  const int D_begin = __ldg(p.D_offsets + t);
  const int D = __ldg(p.D_offsets + t + 1) - D_begin;
  const int64_t row_bytes = static_cast<int64_t>(D) * sizeof(WT);
  const char* table = p.dev_weights + __ldg(p.weights_offsets + t) * static_cast<int64_t>(sizeof(WT));
  const int64_t num_rows = p.rows_per_table ? __ldg(p.rows_per_table + t) : -1;
  const int64_t start = load_index<IndexT>(p.offsets, bag);
  const int64_t end = load_index<IndexT>(p.offsets, bag + 1);

  const int dest = static_cast<int>(b / p.rows_per_dest);
  const int64_t dest_row = b - dest * p.rows_per_dest;
  OT* out = static_cast<OT*>(p.outputs[dest]) + dest_row * p.output_stride + p.output_col_offset +
            D_begin;

  float acc[kVPL][kE];
#pragma unroll
  for (int k = 0; k < kVPL; ++k)
#pragma unroll
    for (int e = 0; e < kE; ++e) acc[k][e] = 0.f;

  const bool weighted = p.per_sample_weights != nullptr;
  const bool vector_rows = (row_bytes & 15) == 0 && (reinterpret_cast<uintptr_t>(table) & 15) == 0;

  if (vector_rows) {
    const int row_vecs = static_cast<int>(row_bytes >> 4);
    const int gs = lanes_per_row(row_vecs);
    const int g = lane / gs;
    const int v = lane - g * gs;
    pool_vector_rows<WT, IndexT, kVPL, kUnroll>(acc, table, row_bytes, row_vecs, gs, p.indices,
                                                p.per_sample_weights, start, end, num_rows,
                                                p.status, lane);
    // combine the groups (gs < 32 implies a single vector per lane)
    for (int o = 16; o >= gs; o >>= 1) {
#pragma unroll
      for (int e = 0; e < kE; ++e) acc[0][e] += __shfl_xor_sync(kFullMask, acc[0][e], o);
    }
    float scale = 1.f;
    if (p.pooling_mode == B200TBE_POOL_MEAN && end > start) scale = 1.f / static_cast<float>(end - start);
    if (g == 0) {
#pragma unroll
      for (int k = 0; k < kVPL; ++k) {
        const int vv = k * 32 + v;
        if (vv < row_vecs) {
          float r[kE];
#pragma unroll
          for (int e = 0; e < kE; ++e) r[e] = acc[k][e] * scale;
          store_pooled<OT, kE>(out + vv * kE, r);
        }
      }
    }
  } else {
    // Rows that are not whole 16-byte vectors: element e of the row lives in lane e % 32.
    float* facc = &acc[0][0];
    for (int64_t c = start; c < end; ++c) {
      const int64_t idx = load_index<IndexT>(p.indices, c);
      const float w = weighted ? __ldg(p.per_sample_weights + c) : 1.f;
      if (num_rows >= 0 && (idx < 0 || idx >= num_rows)) {
        if (lane == 0) atomicOr(p.status, B200TBE_DEV_INDEX_OUT_OF_RANGE);
        continue;
      }
      const char* row = table + idx * row_bytes;
#pragma unroll
      for (int i = 0; i < kVPL * kE; ++i) {
        const int e = i * 32 + lane;
        if (e < D) facc[i] = fmaf(RowVec<WT>::scalar(row + e * sizeof(WT)), w, facc[i]);
      }
    }
    float scale = 1.f;
    if (p.pooling_mode == B200TBE_POOL_MEAN && end > start) scale = 1.f / static_cast<float>(end - start);
#pragma unroll
    for (int i = 0; i < kVPL * kE; ++i) {
      const int e = i * 32 + lane;
      if (e < D) out[e] = to_out(facc[i] * scale, static_cast<OT*>(nullptr));
    }
  }
}

template <typename WT, typename OT, typename IndexT>
int launch_forward(const FwdDev& d, int64_t max_row_bytes, cudaStream_t stream) {
  const int64_t bags = static_cast<int64_t>(d.T) * d.B;
  const int64_t ctas = (bags + kFwdWarps - 1) / kFwdWarps;
  if (ctas > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  const unsigned grid = static_cast<unsigned>(ctas);
  const int64_t vecs = (max_row_bytes + 15) / 16;
  if (vecs <= 32) {
    tbe_forward_kernel<WT, OT, IndexT, 1><<<grid, kFwdThreads, 0, stream>>>(d);
  } else if (vecs <= 64) {
    tbe_forward_kernel<WT, OT, IndexT, 2><<<grid, kFwdThreads, 0, stream>>>(d);
  } else if (vecs <= 128) {
    tbe_forward_kernel<WT, OT, IndexT, 4><<<grid, kFwdThreads, 0, stream>>>(d);
  } else if (vecs <= 256) {
    tbe_forward_kernel<WT, OT, IndexT, 8><<<grid, kFwdThreads, 0, stream>>>(d);
  } else {
    return B200TBE_ERR_UNSUPPORTED;
  }
  return launch_status();
}

template <typename WT, typename OT>
int dispatch_index(const FwdDev& d, int64_t max_row_bytes, int index_bytes, cudaStream_t stream) {
  if (index_bytes == 8) return launch_forward<WT, OT, int64_t>(d, max_row_bytes, stream);
  return launch_forward<WT, OT, int32_t>(d, max_row_bytes, stream);
}

}  // namespace
}  // namespace b200tbe

using namespace b200tbe;

extern "C" int b200tbe_forward(const b200tbe_forward_params* p, b200tbe_stream_t stream_) {
  if (p == nullptr) return B200TBE_ERR_BAD_ARG;
  if (p->T < 0 || p->B < 0 || p->max_D < 0) return B200TBE_ERR_BAD_ARG;
  if (p->T == 0 || p->B == 0) return B200TBE_OK;
  if (p->dev_weights == nullptr || p->weights_offsets == nullptr || p->D_offsets == nullptr ||
      p->offsets == nullptr)
    return B200TBE_ERR_BAD_ARG;
  if (p->index_bytes != 4 && p->index_bytes != 8) return B200TBE_ERR_BAD_ARG;
  if (p->num_dests < 1 || p->num_dests > B200TBE_MAX_DESTS) return B200TBE_ERR_BAD_ARG;
  if (p->rows_per_dest < 1 || p->rows_per_dest * p->num_dests < p->B) return B200TBE_ERR_BAD_ARG;
  if (p->rows_per_table != nullptr && p->status == nullptr) return B200TBE_ERR_BAD_ARG;
  if (p->pooling_mode != B200TBE_POOL_SUM && p->pooling_mode != B200TBE_POOL_MEAN)
    return B200TBE_ERR_UNSUPPORTED;
  FwdDev d;
  d.dev_weights = static_cast<const char*>(p->dev_weights);
  d.weights_offsets = p->weights_offsets;
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
  d.pooling_mode = p->pooling_mode;
  d.status = p->status;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int w = p->weights_dtype, o = p->output_dtype;
  if (w == B200TBE_FP32 && o == B200TBE_FP32)
    return dispatch_index<float, float>(d, int64_t{p->max_D} * 4, p->index_bytes, stream);
  if (w == B200TBE_FP32 && o == B200TBE_FP16)
    return dispatch_index<float, __half>(d, int64_t{p->max_D} * 4, p->index_bytes, stream);
  if (w == B200TBE_FP16 && o == B200TBE_FP32)
    return dispatch_index<__half, float>(d, int64_t{p->max_D} * 2, p->index_bytes, stream);
  if (w == B200TBE_FP16 && o == B200TBE_FP16)
    return dispatch_index<__half, __half>(d, int64_t{p->max_D} * 2, p->index_bytes, stream);
  return B200TBE_ERR_UNSUPPORTED;
}
