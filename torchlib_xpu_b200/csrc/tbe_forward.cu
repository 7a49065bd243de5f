// TBE pooled forward over fp32 / fp16 tables.
//
// Rows of up to 512 bytes (every D <= 128 fp32 / D <= 256 fp16): the register gather of tbe_bags.cuh,
// one warp per group of bags in a plain grid of one-warp CTAs. Wider rows run on the shared-memory ring
// engine of tbe_stream.cuh (persistent, one CTA per SM); rows that are not whole aligned 16-byte
// vectors on a scalar path.
#include "tbe_bags.cuh"

namespace b200tbe {
namespace {

struct FwdParams {
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
  int32_t bags_per_unit;
  int32_t units_per_table;
  int64_t num_units;
  int32_t bag_group;          // bags per warp of the register-gather kernel
  int32_t groups_per_table;
};

// kVPL: vectors of 4 elements a lane may hold (rows of up to 128 * kVPL elements).
template <typename WT, typename OT, typename IndexT, int kVPL>
__global__ void __launch_bounds__(kStreamThreads, 1)
    tbe_forward_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  WarpRing* rings = reinterpret_cast<WarpRing*>(smem_raw);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  WarpRing& ring = rings[warp];
  const StreamBags bags{p.indices, p.offsets, p.per_sample_weights, p.status, p.pooling_mode};
  const int64_t stride_units = static_cast<int64_t>(gridDim.x) * kStreamWarps;
  for (int64_t unit = static_cast<int64_t>(blockIdx.x) * kStreamWarps + warp; unit < p.num_units;
       unit += stride_units) {
    const int t = static_cast<int>(unit / p.units_per_table);
    const int b0 = static_cast<int>(unit - static_cast<int64_t>(t) * p.units_per_table) * p.bags_per_unit;
    const int nb = p.B - b0 < p.bags_per_unit ? p.B - b0 : p.bags_per_unit;
    const int D_begin = __ldg(p.D_offsets + t);
    const int D = __ldg(p.D_offsets + t + 1) - D_begin;
    const int64_t row_bytes = static_cast<int64_t>(D) * sizeof(WT);
    const char* table = p.dev_weights + __ldg(p.weights_offsets + t) * static_cast<int64_t>(sizeof(WT));
    const int64_t num_rows = p.rows_per_table ? __ldg(p.rows_per_table + t) : -1;
    const int64_t bag0 = static_cast<int64_t>(t) * p.B + b0;
    const int64_t col = p.output_col_offset + D_begin;
    OT* const* outputs = reinterpret_cast<OT* const*>(p.outputs);
    const bool streamable = (D & 3) == 0 && (row_bytes & 15) == 0 &&
                            (reinterpret_cast<uintptr_t>(table) & 15) == 0 &&
                            row_bytes <= kStageBytes && (D >> 2) <= 32 * kVPL && D > 0;
    if (streamable) {
      const StreamTable tab{table, row_bytes, static_cast<int>(row_bytes), D >> 2, num_rows};
      const StreamOut<OT> out{outputs, p.output_stride, col, p.rows_per_dest};
      stream_unit<FloatRow<WT>, OT, IndexT, kVPL>(bags, tab, out, bag0, b0, nb, ring, lane);
    } else {
      pool_unit_generic<OT, IndexT>(p.indices, p.offsets, p.per_sample_weights, p.status,
                                    p.pooling_mode, sizeof(WT) == 4 ? B200TBE_FP32 : B200TBE_FP16,
                                    table, row_bytes, D, num_rows, outputs, p.output_stride, col,
                                    p.rows_per_dest, bag0, b0, nb, lane);
    }
  }
}

template <typename WT, typename OT, typename IndexT, bool kWeighted>
__global__ void __launch_bounds__(32, kBagCtasPerSm)
    tbe_forward_bags_kernel(const __grid_constant__ FwdParams p) {
  const int lane = threadIdx.x;
  const int64_t bag = blockIdx.x;
  const int t = static_cast<int>(bag / p.B);
  const int b = static_cast<int>(bag - static_cast<int64_t>(t) * p.B);
  const int D_begin = __ldg(p.D_offsets + t);
  const int D = __ldg(p.D_offsets + t + 1) - D_begin;
  const int row_bytes = D * static_cast<int>(sizeof(WT));
  const char* table = p.dev_weights + __ldg(p.weights_offsets + t) * static_cast<int64_t>(sizeof(WT));
  const int64_t num_rows = p.rows_per_table ? __ldg(p.rows_per_table + t) : -1;
  OT* const* outputs = reinterpret_cast<OT* const*>(p.outputs);
  if ((row_bytes & 15) != 0 || (reinterpret_cast<uintptr_t>(table) & 15) != 0 || row_bytes > 512 ||
      D <= 0) {
    pool_unit_generic<OT, IndexT>(p.indices, p.offsets, p.per_sample_weights, p.status,
                                  p.pooling_mode, sizeof(WT) == 4 ? B200TBE_FP32 : B200TBE_FP16,
                                  table, row_bytes, D, num_rows, outputs, p.output_stride,
                                  p.output_col_offset + D_begin, p.rows_per_dest, bag, b, 1, lane);
    return;
  }
  const BagLaunch<OT> launch{p.indices, p.offsets, p.per_sample_weights, p.status, p.pooling_mode,
                             outputs, p.output_stride, p.rows_per_dest};
  pool_float_bag<WT, OT, IndexT, kWeighted>(launch, table, row_bytes, num_rows,
                                            p.output_col_offset + D_begin, bag, b, lane);
}

// Per-sample weights travel with the rows and take the kernel to 85 registers: 24 CTAs per SM then
// (26 tables x 8192 weighted bags: 0.215 ms; 0.228 ms at 32 CTAs with spills, 0.236 at 28).
template <typename WT, typename OT, typename IndexT, bool kWeighted>
__global__ void __launch_bounds__(32, kWeighted ? 24 : kBagCtasPerSm)
    tbe_forward_bag_groups_kernel(const __grid_constant__ FwdParams p) {
  const int lane = threadIdx.x;
  const int t = static_cast<int>(blockIdx.x / static_cast<unsigned>(p.groups_per_table));
  const int b0 = static_cast<int>(blockIdx.x - static_cast<unsigned>(t) * p.groups_per_table) * p.bag_group;
  const int nb = p.B - b0 < p.bag_group ? p.B - b0 : p.bag_group;
  const int64_t bag0 = static_cast<int64_t>(t) * p.B + b0;
  const int D_begin = __ldg(p.D_offsets + t);
  const int D = __ldg(p.D_offsets + t + 1) - D_begin;
  const int row_bytes = D * static_cast<int>(sizeof(WT));
  const char* table = p.dev_weights + __ldg(p.weights_offsets + t) * static_cast<int64_t>(sizeof(WT));
  const int64_t num_rows = p.rows_per_table ? __ldg(p.rows_per_table + t) : -1;
  OT* const* outputs = reinterpret_cast<OT* const*>(p.outputs);
  if ((row_bytes & 15) != 0 || (reinterpret_cast<uintptr_t>(table) & 15) != 0 || row_bytes > 512 ||
      D <= 0) {
    pool_unit_generic<OT, IndexT>(p.indices, p.offsets, p.per_sample_weights, p.status,
                                  p.pooling_mode, sizeof(WT) == 4 ? B200TBE_FP32 : B200TBE_FP16,
                                  table, row_bytes, D, num_rows, outputs, p.output_stride,
                                  p.output_col_offset + D_begin, p.rows_per_dest, bag0, b0, nb, lane);
    return;
  }
  const BagLaunch<OT> launch{p.indices, p.offsets, p.per_sample_weights, p.status, p.pooling_mode,
                             outputs, p.output_stride, p.rows_per_dest};
  pool_float_bags<WT, OT, IndexT, kWeighted>(launch, table, row_bytes, num_rows,
                                             p.output_col_offset + D_begin, bag0, b0, nb, lane);
}

template <typename WT, typename OT, typename IndexT>
int launch_bags(const FwdParams& d0, cudaStream_t stream) {
  const int64_t bags = static_cast<int64_t>(d0.T) * d0.B;
  if (bags > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  FwdParams d = d0;
  d.bag_group = bag_group_for(bags);
  d.groups_per_table = (d.B + d.bag_group - 1) / d.bag_group;
  const unsigned grid = static_cast<unsigned>(static_cast<int64_t>(d.T) * d.groups_per_table);
  const bool weighted = d.per_sample_weights != nullptr;
  if (d.bag_group == 1) {
    if (weighted)
      tbe_forward_bags_kernel<WT, OT, IndexT, true><<<grid, 32, 0, stream>>>(d);
    else
      tbe_forward_bags_kernel<WT, OT, IndexT, false><<<grid, 32, 0, stream>>>(d);
  } else {
    if (weighted)
      tbe_forward_bag_groups_kernel<WT, OT, IndexT, true><<<grid, 32, 0, stream>>>(d);
    else
      tbe_forward_bag_groups_kernel<WT, OT, IndexT, false><<<grid, 32, 0, stream>>>(d);
  }
  return launch_status();
}

template <typename WT, typename OT, typename IndexT, int kVPL>
int launch_one(const FwdParams& d, cudaStream_t stream) {
  auto kernel = tbe_forward_kernel<WT, OT, IndexT, kVPL>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kStreamSmemBytes)) != cudaSuccess)
    return B200TBE_ERR_LAUNCH;
  const int64_t ctas = (d.num_units + kStreamWarps - 1) / kStreamWarps;
  const unsigned grid = static_cast<unsigned>(ctas < kNumSMs ? ctas : kNumSMs);
  kernel<<<grid, kStreamThreads, kStreamSmemBytes, stream>>>(d);
  return launch_status();
}

template <typename WT, typename OT, typename IndexT>
int launch_forward(const FwdParams& d, int max_D, cudaStream_t stream) {
  if (static_cast<int64_t>(max_D) * sizeof(WT) <= 512) return launch_bags<WT, OT, IndexT>(d, stream);
  if (max_D <= 128) return launch_one<WT, OT, IndexT, 1>(d, stream);
  if (max_D <= 256) return launch_one<WT, OT, IndexT, 2>(d, stream);
  if (max_D <= 512) return launch_one<WT, OT, IndexT, 4>(d, stream);
  if (max_D <= 1024) return launch_one<WT, OT, IndexT, 8>(d, stream);
  return B200TBE_ERR_UNSUPPORTED;
}

template <typename WT, typename OT>
int dispatch_index(const FwdParams& d, int max_D, int index_bytes, cudaStream_t stream) {
  if (index_bytes == 8) return launch_forward<WT, OT, int64_t>(d, max_D, stream);
  return launch_forward<WT, OT, int32_t>(d, max_D, stream);
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
  FwdParams d;
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
  d.bags_per_unit = stream_bags_per_unit(p->T, p->B);
  d.units_per_table = (p->B + d.bags_per_unit - 1) / d.bags_per_unit;
  d.num_units = static_cast<int64_t>(p->T) * d.units_per_table;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int w = p->weights_dtype, o = p->output_dtype;
  if (w == B200TBE_FP32 && o == B200TBE_FP32)
    return dispatch_index<float, float>(d, p->max_D, p->index_bytes, stream);
  if (w == B200TBE_FP32 && o == B200TBE_FP16)
    return dispatch_index<float, __half>(d, p->max_D, p->index_bytes, stream);
  if (w == B200TBE_FP16 && o == B200TBE_FP32)
    return dispatch_index<__half, float>(d, p->max_D, p->index_bytes, stream);
  if (w == B200TBE_FP16 && o == B200TBE_FP16)
    return dispatch_index<__half, __half>(d, p->max_D, p->index_bytes, stream);
  return B200TBE_ERR_UNSUPPORTED;
}
