// TBE pooled forward over fp32 / fp16 tables.
//
// Rows of up to 512 bytes (every D <= 128 fp32 / D <= 256 fp16): one warp per bag, launched as a
// plain grid of bags with few registers per thread, so that ~48 warps are resident per SM and the
// hardware's CTA scheduling balances the load. Measured on B200 this simple shape beats both a
// persistent software-pipelined variant and the shared-memory ring engine (which stops at ~19 G
// rows/s for 256-byte rows): a random-row read kernel reaches 28 G rows/s out of HBM and 51 G
// rows/s out of L2 only at high occupancy. A row of C 16-byte vectors is fetched by a group of gs
// lanes (C rounded up to a power of two), so one load instruction brings 32/gs rows (two 256-byte
// rows); the bag's ids are read 32 at a time with one coalesced load and handed out by shuffle as
// 32-bit chunk numbers; loads allocate in L1, where the hottest rows of a skewed id stream hit;
// fp16 elements are added to fp32 accumulators with the mixed-precision add of sm_100.
// Wider rows run on the ring engine of tbe_stream.cuh; rows that are not whole aligned 16-byte
// vectors on a scalar path.
#include "tbe_stream.cuh"

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
};

// kVPL: vectors of 4 elements a lane may hold (rows of up to 128 * kVPL elements).
template <typename WT, typename OT, typename IndexT, int kVPL>
__global__ void __launch_bounds__(kStreamThreads, 1)
    tbe_forward_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  WarpRing* rings = reinterpret_cast<WarpRing*>(smem_raw);
  stream_init_rings(rings);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  WarpRing& ring = rings[warp];
  uint32_t phases = 0;
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
      if (!stream_unit<FloatRow<WT>, OT, IndexT, kVPL>(bags, tab, out, bag0, b0, nb, ring, phases, lane))
        return;
    } else {
      pool_unit_generic<OT, IndexT>(p.indices, p.offsets, p.per_sample_weights, p.status,
                                    p.pooling_mode, sizeof(WT) == 4 ? B200TBE_FP32 : B200TBE_FP16,
                                    table, row_bytes, D, num_rows, outputs, p.output_stride, col,
                                    p.rows_per_dest, bag0, b0, nb, lane);
    }
  }
}

// ---- one warp per bag, rows of at most 512 bytes ---------------------------------------------
constexpr int kBagWarps = 8;
constexpr int kBagThreads = kBagWarps * 32;
constexpr int kBagCtasPerSm = 8;   // 64 warps per SM, 32 registers per thread: measured best (5: +20 %, 6: +21 %)
constexpr int kBagLoads = 2;       // 16-byte loads in flight per lane
constexpr uint32_t kNoRow = 0xffffffffu;

__device__ __forceinline__ uint4 ldg_cached16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// acc[0..1] += the two fp16 halves of one 32-bit word, one mixed-precision add each.
__device__ __forceinline__ void add_half2(float& a0, float& a1, uint32_t h2) {
  asm("{.reg .f16 l, h;\n"
      "mov.b32 {l, h}, %2;\n"
      "add.rn.f32.f16 %0, l, %0;\n"
      "add.rn.f32.f16 %1, h, %1;}\n"
      : "+f"(a0), "+f"(a1)
      : "r"(h2));
}

template <typename WT>
struct Vec16;
template <>
struct Vec16<float> {
  static constexpr int kE = 4;
  static __device__ __forceinline__ void add(float (&a)[4], uint4 x) {
    a[0] += __uint_as_float(x.x);
    a[1] += __uint_as_float(x.y);
    a[2] += __uint_as_float(x.z);
    a[3] += __uint_as_float(x.w);
  }
  static __device__ __forceinline__ void fma(float (&a)[4], uint4 x, float w) {
    a[0] = fmaf(__uint_as_float(x.x), w, a[0]);
    a[1] = fmaf(__uint_as_float(x.y), w, a[1]);
    a[2] = fmaf(__uint_as_float(x.z), w, a[2]);
    a[3] = fmaf(__uint_as_float(x.w), w, a[3]);
  }
};
template <>
struct Vec16<__half> {
  static constexpr int kE = 8;
  static __device__ __forceinline__ void add(float (&a)[8], uint4 x) {
    add_half2(a[0], a[1], x.x);
    add_half2(a[2], a[3], x.y);
    add_half2(a[4], a[5], x.z);
    add_half2(a[6], a[7], x.w);
  }
  static __device__ __forceinline__ void fma(float (&a)[8], uint4 x, float w) {
    const float2 p0 = half2_bits_to_float2(x.x), p1 = half2_bits_to_float2(x.y),
                 p2 = half2_bits_to_float2(x.z), p3 = half2_bits_to_float2(x.w);
    a[0] = fmaf(p0.x, w, a[0]);
    a[1] = fmaf(p0.y, w, a[1]);
    a[2] = fmaf(p1.x, w, a[2]);
    a[3] = fmaf(p1.y, w, a[3]);
    a[4] = fmaf(p2.x, w, a[4]);
    a[5] = fmaf(p2.y, w, a[5]);
    a[6] = fmaf(p3.x, w, a[6]);
    a[7] = fmaf(p3.y, w, a[7]);
  }
};

template <typename WT, typename OT, typename IndexT, bool kWeighted>
__global__ void __launch_bounds__(kBagThreads, kBagCtasPerSm)
    tbe_forward_bags_kernel(const __grid_constant__ FwdParams p) {
  constexpr int kE = Vec16<WT>::kE;
  const int lane = threadIdx.x & 31;
  const int64_t bag = static_cast<int64_t>(blockIdx.x) * kBagWarps + (threadIdx.x >> 5);
  if (bag >= static_cast<int64_t>(p.T) * p.B) return;
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
  const int64_t start = load_index<IndexT>(p.offsets, bag);
  const int64_t end = load_index<IndexT>(p.offsets, bag + 1);
  const int len = end - start > 0x7fffffff ? 0x7fffffff : static_cast<int>(end - start);
  const IndexT* idx = reinterpret_cast<const IndexT*>(p.indices) + start;
  const float* psw = kWeighted ? p.per_sample_weights + start : nullptr;
  const int vecs = row_bytes >> 4;
  const int gs = lanes_per_row(vecs);
  const int gshift = __ffs(gs) - 1;
  const int G = 32 >> gshift;            // rows per load instruction
  const int h = lane >> gshift;          // this lane's group
  const int v = lane & (gs - 1);         // this lane's vector inside the row
  const bool active = v < vecs;
  const char* lane_base = table + (v << 4);

  float acc[kE];
#pragma unroll
  for (int e = 0; e < kE; ++e) acc[e] = 0.f;

  for (int c = 0; c < len; c += 32) {
    const int n = len - c < 32 ? len - c : 32;
    // this lane's row id; ids do not fit 32 bits only in tables no memory holds
    uint32_t my_row = kNoRow;
    float my_w = 1.f;
    if (lane < n) {
      const int64_t i = static_cast<int64_t>(__ldg(idx + c + lane));
      if (kWeighted) my_w = __ldg(psw + c + lane);
      if (i < 0 || i >= (num_rows >= 0 ? num_rows : int64_t{0xffffffff})) {
        if (p.status != nullptr) atomicOr(p.status, B200TBE_DEV_INDEX_OUT_OF_RANGE);
      } else {
        my_row = static_cast<uint32_t>(i);
      }
    }
    for (int j = 0; j < n; j += G * kBagLoads) {
      uint4 x[kBagLoads];
      float w[kBagLoads];
#pragma unroll
      for (int u = 0; u < kBagLoads; ++u) {
        const int rr = j + u * G + h;
        const uint32_t row = __shfl_sync(kFullMask, my_row, rr & 31);
        if (kWeighted) w[u] = __shfl_sync(kFullMask, my_w, rr & 31);
        x[u] = make_uint4(0u, 0u, 0u, 0u);  // +0.0 in either type: adding it changes nothing
        if (rr < n && row != kNoRow && active)
          x[u] = ldg_cached16(lane_base + static_cast<uint64_t>(row) * static_cast<uint32_t>(row_bytes));
      }
#pragma unroll
      for (int u = 0; u < kBagLoads; ++u) {
        if (kWeighted) {
          Vec16<WT>::fma(acc, x[u], w[u]);
        } else {
          Vec16<WT>::add(acc, x[u]);
        }
      }
    }
  }
  for (int o = gs; o < 32; o <<= 1) {
#pragma unroll
    for (int e = 0; e < kE; ++e) acc[e] += __shfl_xor_sync(kFullMask, acc[e], o);
  }
  if (h == 0 && active) {
    const float scale =
        (p.pooling_mode == B200TBE_POOL_MEAN && len > 0) ? 1.f / static_cast<float>(len) : 1.f;
    const int rpd = static_cast<int>(p.rows_per_dest);
    const int dest = b / rpd;
    OT* dst = outputs[dest] + static_cast<int64_t>(b - dest * rpd) * p.output_stride +
              p.output_col_offset + D_begin + v * kE;
    float r[kE];
#pragma unroll
    for (int e = 0; e < kE; ++e) r[e] = acc[e] * scale;
#pragma unroll
    for (int e = 0; e < kE; e += 4) store_pooled<OT, 4>(dst + e, r + e);
  }
}

template <typename WT, typename OT, typename IndexT>
int launch_bags(const FwdParams& d, cudaStream_t stream) {
  const int64_t bags = static_cast<int64_t>(d.T) * d.B;
  const int64_t ctas = (bags + kBagWarps - 1) / kBagWarps;
  if (ctas > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  const unsigned grid = static_cast<unsigned>(ctas);
  if (d.per_sample_weights != nullptr) {
    tbe_forward_bags_kernel<WT, OT, IndexT, true><<<grid, kBagThreads, 0, stream>>>(d);
  } else {
    tbe_forward_bags_kernel<WT, OT, IndexT, false><<<grid, kBagThreads, 0, stream>>>(d);
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
