// Quantised-inference TBE forward: INT8 / INT4 / INT2 row-wise quantised tables with an fp16
// {scale, bias} header per row, plus FP16 / FP32 tables, mixed per table.
//
// Two kernels share a call. INT8 and INT4 tables of at most 128 elements per row -- what inference
// tables are -- go through the register gather of tbe_nbit_bags.cuh (one warp per group of bags, code words
// fetched straight into registers). Everything else (INT2, float rows, wider rows, rows that are
// not 4-byte aligned) goes through the streaming gather engine of tbe_stream.cuh, described next;
// each kernel skips the other's tables.
//
// A whole row (header + payload, rounded up to 16 bytes) is brought to shared memory. The consuming
// warp reads it one row per instruction: every lane loads the 4-byte header (a shared-memory
// broadcast) and the bytes of its own 4 elements (4, 2 or 1 bytes for INT8, INT4, INT2), so all 32
// lanes dequantise payload for D = 128 regardless of the 4-byte header that misaligns the payload
// in global memory. q * (scale * weight) is accumulated per element in fp32 and bias * weight once
// per row; the bias sum is added when the bag is written.
//
#include "tbe_bags.cuh"

namespace b200tbe {
namespace {

struct NbitParams {
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
  int32_t bags_per_unit;
  int32_t units_per_table;
  int64_t num_units;
  int32_t only_bag_tables;   // the caller vouches that every table is INT8 / INT4: no ring kernel
  int32_t bag_group;         // bags per warp of the register-gather kernel
  int32_t groups_per_table;
};

__device__ __forceinline__ int64_t round_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

// Bytes of a row's header and payload, and the distance between rows.
__device__ __forceinline__ void nbit_row_geometry(int ty, int D, int row_alignment, int& header,
                                                  int64_t& payload, int64_t& row_stride) {
  header = 4;
  switch (ty) {
    case B200TBE_INT8: payload = D; break;
    case B200TBE_INT4: payload = (D + 1) / 2; break;
    case B200TBE_INT2: payload = (D + 3) / 4; break;
    case B200TBE_FP16: payload = int64_t{D} * 2; header = 0; break;
    default: payload = int64_t{D} * 4; header = 0; break;
  }
  row_stride = round_up(header + payload, row_alignment);
}
__device__ __forceinline__ int64_t nbit_row_stride(int ty, int D, int row_alignment) {
  int header;
  int64_t payload, stride;
  nbit_row_geometry(ty, D, row_alignment, header, payload, stride);
  return stride;
}

#include "tbe_nbit_bags.cuh"

template <typename OT, typename IndexT, int kVPL>
__global__ void __launch_bounds__(kStreamThreads, 1)
    tbe_nbit_forward_kernel(const __grid_constant__ NbitParams p) {
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
    const int ty = __ldg(p.weights_tys + t);
    const int D_begin = __ldg(p.D_offsets + t);
    const int D = __ldg(p.D_offsets + t + 1) - D_begin;
    const char* table = reinterpret_cast<const char*>(p.dev_weights) + __ldg(p.weights_offsets + t);
    const int64_t num_rows = p.rows_per_table ? __ldg(p.rows_per_table + t) : -1;
    const int64_t bag0 = static_cast<int64_t>(t) * p.B + b0;
    const int64_t col = p.output_col_offset + D_begin;
    OT* const* outputs = reinterpret_cast<OT* const*>(p.outputs);

    int64_t payload, row_stride;
    int header;
    nbit_row_geometry(ty, D, p.row_alignment, header, payload, row_stride);
    if (nbit_bag_path(ty, D, table, row_stride)) continue;   // pooled by tbe_nbit_bags_kernel
    const int64_t copy_bytes = round_up(header + payload, 16);
    const bool streamable = (D & 3) == 0 && D > 0 && (row_stride & 15) == 0 &&
                            (reinterpret_cast<uintptr_t>(table) & 15) == 0 &&
                            copy_bytes <= row_stride && copy_bytes <= kStageBytes &&
                            (D >> 2) <= 32 * kVPL;
    if (streamable) {
      const StreamTable tab{table, row_stride, static_cast<int>(copy_bytes), D >> 2, num_rows};
      const StreamOut<OT> out{outputs, p.output_stride, col, p.rows_per_dest};
      switch (ty) {
        case B200TBE_INT8:
          stream_unit<QuantRow<8>, OT, IndexT, kVPL>(bags, tab, out, bag0, b0, nb, ring, lane);
          break;
        case B200TBE_INT4:
          stream_unit<QuantRow<4>, OT, IndexT, kVPL>(bags, tab, out, bag0, b0, nb, ring, lane);
          break;
        case B200TBE_INT2:
          stream_unit<QuantRow<2>, OT, IndexT, kVPL>(bags, tab, out, bag0, b0, nb, ring, lane);
          break;
        case B200TBE_FP16:
          stream_unit<FloatRow<__half>, OT, IndexT, kVPL>(bags, tab, out, bag0, b0, nb, ring, lane);
          break;
        default:
          stream_unit<FloatRow<float>, OT, IndexT, kVPL>(bags, tab, out, bag0, b0, nb, ring, lane);
          break;
      }
    } else {
      pool_unit_generic<OT, IndexT>(p.indices, p.offsets, p.per_sample_weights, p.status,
                                    p.pooling_mode, ty, table, row_stride, D, num_rows, outputs,
                                    p.output_stride, col, p.rows_per_dest, bag0, b0, nb, lane);
    }
  }
}

template <typename OT, typename IndexT, int kVPL>
int launch_one(const NbitParams& d, cudaStream_t stream) {
  auto kernel = tbe_nbit_forward_kernel<OT, IndexT, kVPL>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kStreamSmemBytes)) != cudaSuccess)
    return B200TBE_ERR_LAUNCH;
  const int64_t ctas = (d.num_units + kStreamWarps - 1) / kStreamWarps;
  const unsigned grid = static_cast<unsigned>(ctas < kNumSMs ? ctas : kNumSMs);
  kernel<<<grid, kStreamThreads, kStreamSmemBytes, stream>>>(d);
  return launch_status();
}

template <typename OT, typename IndexT>
int launch_bags(const NbitParams& d0, cudaStream_t stream) {
  const int64_t bags = static_cast<int64_t>(d0.T) * d0.B;
  if (bags > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  NbitParams d = d0;
  // bags of quantised tables are long (a hundred lookups), so small groups already keep the rounds
  // full: 64 tables x 16384 bags run in 2.05 / 1.83 / 1.71 / 1.66 / 1.67 / 1.72 ms for groups of
  // 1 / 2 / 4 / 8 / 16 / 32
  d.bag_group = bag_group_for(bags) < 8 ? bag_group_for(bags) : 8;
  d.groups_per_table = (d.B + d.bag_group - 1) / d.bag_group;
  const int64_t ctas = static_cast<int64_t>(d.T) * d.groups_per_table;
  if (d.per_sample_weights != nullptr)
    tbe_nbit_bags_kernel<OT, IndexT, true><<<static_cast<unsigned>(ctas), kNbitBagThreads, 0, stream>>>(d);
  else
    tbe_nbit_bags_kernel<OT, IndexT, false><<<static_cast<unsigned>(ctas), kNbitBagThreads, 0, stream>>>(d);
  return launch_status();
}

template <typename OT, typename IndexT>
int launch_nbit(const NbitParams& d, int max_D, cudaStream_t stream) {
  const int st = launch_bags<OT, IndexT>(d, stream);
  if (st != B200TBE_OK || d.only_bag_tables) return st;
  if (max_D <= 128) return launch_one<OT, IndexT, 1>(d, stream);
  if (max_D <= 256) return launch_one<OT, IndexT, 2>(d, stream);
  if (max_D <= 512) return launch_one<OT, IndexT, 4>(d, stream);
  return launch_one<OT, IndexT, 8>(d, stream);  // wider rows take the generic path per table
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
  NbitParams d;
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
  d.bags_per_unit = stream_bags_per_unit(p->T, p->B);
  d.units_per_table = (p->B + d.bags_per_unit - 1) / d.bags_per_unit;
  d.num_units = static_cast<int64_t>(p->T) * d.units_per_table;
  // types present, when the caller says (bit i: some table has type code i): with INT8 and INT4
  // alone and narrow rows the ring kernel would find nothing to do and is not launched
  const uint32_t fast_types = (1u << B200TBE_INT8) | (1u << B200TBE_INT4);
  d.only_bag_tables = p->table_type_mask != 0 && (p->table_type_mask & ~fast_types) == 0 &&
                      p->max_D <= kNbitBagMaxD && p->row_alignment % 4 == 0;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const bool i64 = p->index_bytes == 8;
  if (p->output_dtype == B200TBE_FP32)
    return i64 ? launch_nbit<float, int64_t>(d, p->max_D, stream)
               : launch_nbit<float, int32_t>(d, p->max_D, stream);
  if (p->output_dtype == B200TBE_FP16)
    return i64 ? launch_nbit<__half, int64_t>(d, p->max_D, stream)
               : launch_nbit<__half, int32_t>(d, p->max_D, stream);
  return B200TBE_ERR_UNSUPPORTED;
}
