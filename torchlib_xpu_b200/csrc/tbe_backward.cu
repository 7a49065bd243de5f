// TBE backward with the optimizer fused: exact (one update per distinct row) SGD / row-wise Adagrad.
//
// Rows of up to 512 elements (tbe_backward_sweep.cuh):
//   plan        the lookups of table t are the index range [offsets[t*B], offsets[(t+1)*B]); every
//               table's range is cut into tiles of 4096 lookups, described on the device
//   linearize   key = row id, payload = bag id (or the lookup position when per-sample weights are
//               in use); the table is implied by the position
//   sort        radix_sort.cu, segmented: every table's range is sorted by row on its own, over the
//               bits of the largest table only (22 bits for 4 M rows, whatever the number of tables)
//   sweep       groups of lanes walk spans of 256 sorted lookups, summing gradient slices in
//               registers and updating a row where its run of equal keys ends; since the sorted order
//               is (table, row), only one table's B x D_t slice of the gradient matrix is live in L2
//   finish      runs that cross span boundaries: their per-span partial sums are added in span order
// Wider rows (up to 1024 elements):
//   linearize   key = hash_size_cumsum[t] + index; flat sort over total_hash_size_bits bits
//   segment     head flags + compaction give the start of every run of equal keys
//   reduce      persistent grid, one CTA per SM, on the shared-memory ring engine of tbe_stream.cuh
//               (a warp takes 31 consecutive runs and streams the gradient slices of their lookups
//               through its ring). Runs longer than kLongRun are cut into chunks of kLongRun lookups:
//               a second kernel streams each chunk into a partial row in scratch and a third adds a
//               run's partials in chunk order and applies the update.
// Summation order is fixed by the data alone on both paths.
#include "radix_sort.cuh"
#include "scan.cuh"
#include "tbe_bags.cuh"

namespace b200tbe {
namespace {

constexpr int kBwdWarps = 8;
constexpr int kBwdThreads = kBwdWarps * 32;
constexpr int kLongRun = 256;           // lookups per chunk of a long run
constexpr int kSegThreads = 1024;
constexpr int kSegItems = 4;
constexpr int kSegTile = kSegThreads * kSegItems;
constexpr uint32_t kInvalidPayload = 0xffffffffu;

// Widest digit of the segmented sort's passes: 8 bits (22-bit row ids sort in passes of 8, 7 and
// 7 bits). Measured on the bench step against two passes of 11 bits: the 256-digit scatter runs at
// 0.68 ms per pass, the 2048-digit one at 1.57 ms (its digit tables leave three CTAs per SM and the
// per-tile digit scan is eight times as long).
constexpr int kSweepSortDigitBits = 8;

struct BwdDev {
  char* dev_weights;
  const int64_t* weights_offsets;
  const int32_t* D_offsets;
  const int64_t* hash_size_cumsum;
  const void* indices;
  const void* offsets;
  const float* per_sample_weights;
  const char* grad_output;
  int64_t grad_stride;
  int64_t grad_col_offset;
  float* momentum1;
  const int64_t* momentum1_offsets;
  int64_t num_indices;
  int32_t T;
  int32_t B;
  int32_t pooling_mode;
  int32_t optimizer;
  int32_t index_bytes;
  float learning_rate;
  float eps;
  int32_t* status;
  // scratch
  const void* sorted_keys;
  const uint32_t* sorted_vals;
  uint32_t* bag_of_pos;      // only with per-sample weights
  uint32_t* run_start;       // [num_runs + 1]
  uint32_t* counters;        // [0] runs, [1] long runs, [2] chunks
  uint32_t* long_run;        // [max_long] run id of each long run
  uint32_t* long_chunk0;     // [max_long] first chunk of each long run
  uint32_t* chunk_run;       // [max_chunks] slot (index into long_run) of each chunk
  float* partials;           // [max_chunks][max_D]; sweep path: [2 * spans][max_D] (head, tail slot)
  int32_t max_D;
  // sweep path: the plan (tables -> tiles -> spans)
  const uint32_t* seg_start;       // [T + 1] first sorted position of each table
  const uint32_t* seg_tile_base;   // [T + 1] first tile of each table
  const uint32_t* total_tiles;     // tiles in use
  const uint4* tile_desc;          // [max_tiles] {begin, count, table, first tile of the table}
  uint32_t* span_flags;            // [max_tiles * 16]
};

// ---- linearize -----------------------------------------------------------------------------
// One warp per 32 consecutive bags: lane i holds the start of bag i (relative to the group's first
// lookup) and the bag's table; the group's lookups are then walked 32 at a time, fully coalesced,
// and each lookup finds its bag with a 5-step search over the lanes' starts.
template <typename KeyT, typename IndexT, bool kWeighted>
__global__ void __launch_bounds__(kBwdThreads)
    linearize_kernel(BwdDev p, KeyT* __restrict__ keys, uint32_t* __restrict__ vals) {
  const int lane = threadIdx.x & 31;
  const int64_t total_bags = static_cast<int64_t>(p.T) * p.B;
  const int64_t bag0 = (static_cast<int64_t>(blockIdx.x) * kBwdWarps + (threadIdx.x >> 5)) * 32;
  if (bag0 >= total_bags) return;
  const int nb = total_bags - bag0 < 32 ? static_cast<int>(total_bags - bag0) : 32;
  const int64_t begin = load_index<IndexT>(p.offsets, bag0);
  const int64_t end = load_index<IndexT>(p.offsets, bag0 + nb);
  const int64_t mine = load_index<IndexT>(p.offsets, bag0 + (lane < nb ? lane : nb));
  // a group of 32 bags longer than 2^32 lookups does not occur in memory that exists
  const uint32_t my_start = static_cast<uint32_t>(mine - begin);
  const int my_t = static_cast<int>((bag0 + (lane < nb ? lane : nb - 1)) / p.B);
  const int64_t my_h0 = __ldg(p.hash_size_cumsum + my_t);
  const int64_t my_rows = __ldg(p.hash_size_cumsum + my_t + 1) - my_h0;
  const uint32_t total = static_cast<uint32_t>(end - begin);
  for (uint32_t base = 0; base < total; base += 32) {
    const uint32_t rel = base + lane;
    // the last bag whose start is <= rel (empty bags share a start with their successor)
    int b = 0;
#pragma unroll
    for (int step = 16; step > 0; step >>= 1) {
      const int cand = b + step;
      const uint32_t s = __shfl_sync(kFullMask, my_start, cand & 31);
      if (cand < nb && s <= rel) b = cand;
    }
    const int64_t h0 = __shfl_sync(kFullMask, my_h0, b);
    const int64_t rows = __shfl_sync(kFullMask, my_rows, b);
    if (rel < total) {
      const int64_t j = begin + rel;
      int64_t idx = load_index<IndexT>(p.indices, j);
      const uint32_t bag = static_cast<uint32_t>(bag0 + b);
      uint32_t payload = kWeighted ? static_cast<uint32_t>(j) : bag;
      if (idx < 0 || idx >= rows) {
        if (p.status != nullptr) atomicOr(p.status, B200TBE_DEV_INDEX_OUT_OF_RANGE);
        idx = 0;
        payload = kInvalidPayload;
      }
      keys[j] = static_cast<KeyT>(h0 + idx);
      vals[j] = payload;
      if (kWeighted) p.bag_of_pos[j] = bag;
    }
  }
}

// ---- run-length segmentation --------------------------------------------------------------
template <typename KeyT>
__device__ __forceinline__ bool is_head(const KeyT* keys, int64_t i) {
  return i == 0 || keys[i] != keys[i - 1];
}

template <typename KeyT>
__global__ void __launch_bounds__(kSegThreads)
    count_heads_kernel(const KeyT* __restrict__ keys, int64_t n, uint32_t* __restrict__ tile_heads) {
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kSegTile + threadIdx.x * kSegItems;
  uint32_t c = 0;
#pragma unroll
  for (int i = 0; i < kSegItems; ++i)
    if (base + i < n && is_head(keys, base + i)) ++c;
  uint32_t total;
  block_exclusive_scan(c, &total);
  if (threadIdx.x == 0) tile_heads[blockIdx.x] = total;
}

// tile_heads holds the exclusive scan of the per-tile head counts; counters[0] the total.
template <typename KeyT>
__global__ void __launch_bounds__(kSegThreads)
    write_run_starts_kernel(const KeyT* __restrict__ keys, int64_t n,
                            const uint32_t* __restrict__ tile_heads,
                            const uint32_t* __restrict__ counters, uint32_t* __restrict__ run_start) {
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kSegTile + threadIdx.x * kSegItems;
  bool head[kSegItems];
  uint32_t c = 0;
#pragma unroll
  for (int i = 0; i < kSegItems; ++i) {
    head[i] = base + i < n && is_head(keys, base + i);
    c += head[i] ? 1u : 0u;
  }
  uint32_t total;
  uint32_t at = block_exclusive_scan(c, &total) + tile_heads[blockIdx.x];
#pragma unroll
  for (int i = 0; i < kSegItems; ++i)
    if (head[i]) run_start[at++] = static_cast<uint32_t>(base + i);
  if (blockIdx.x == 0 && threadIdx.x == 0) run_start[counters[0]] = static_cast<uint32_t>(n);
}

__device__ __forceinline__ int64_t bag_length(const BwdDev& p, int64_t bag) {
  if (p.index_bytes == 8)
    return load_index<int64_t>(p.offsets, bag + 1) - load_index<int64_t>(p.offsets, bag);
  return load_index<int32_t>(p.offsets, bag + 1) - load_index<int32_t>(p.offsets, bag);
}

template <typename WT>
__device__ __forceinline__ void update_elems4(WT* w, const float* g, float mult);
template <>
__device__ __forceinline__ void update_elems4<float>(float* w, const float* g, float mult) {
  float4 x = *reinterpret_cast<float4*>(w);
  x.x = fmaf(-mult, g[0], x.x);
  x.y = fmaf(-mult, g[1], x.y);
  x.z = fmaf(-mult, g[2], x.z);
  x.w = fmaf(-mult, g[3], x.w);
  *reinterpret_cast<float4*>(w) = x;
}
template <>
__device__ __forceinline__ void update_elems4<__half>(__half* w, const float* g, float mult) {
  uint2 raw = *reinterpret_cast<uint2*>(w);
  float2 a = half2_bits_to_float2(raw.x), b = half2_bits_to_float2(raw.y);
  a.x = fmaf(-mult, g[0], a.x);
  a.y = fmaf(-mult, g[1], a.y);
  b.x = fmaf(-mult, g[2], b.x);
  b.y = fmaf(-mult, g[3], b.y);
  raw.x = float2_to_half2_bits(a.x, a.y);  // round to nearest even
  raw.y = float2_to_half2_bits(b.x, b.y);
  *reinterpret_cast<uint2*>(w) = raw;
}

// Applies the optimizer to one row given its summed gradient, held by the lanes of group 0
// (lane v < slice_vecs holds elements [v*kE, (v+1)*kE) of vector k).
template <typename WT, int kE, int kVPL>
__device__ __forceinline__ void apply_update(const BwdDev& p, float (&acc)[kVPL][kE], int t,
                                             int64_t row, int D, int gs, int slice_vecs, int lane) {
  const int g = lane / gs;
  const int v = lane - g * gs;
  float mult = p.learning_rate;
  if (p.optimizer == B200TBE_OPT_ROWWISE_ADAGRAD) {
    float sq = 0.f;
    if (g == 0) {
#pragma unroll
      for (int k = 0; k < kVPL; ++k)
        if (k * 32 + v < slice_vecs)
#pragma unroll
          for (int e = 0; e < kE; ++e) sq = fmaf(acc[k][e], acc[k][e], sq);
    }
    sq = warp_sum(sq);
    float* m = p.momentum1 + __ldg(p.momentum1_offsets + t) + row;
    float m_new = 0.f;
    if (lane == 0) {
      m_new = *m + sq / static_cast<float>(D);
      *m = m_new;
    }
    m_new = __shfl_sync(kFullMask, m_new, 0);
    mult = p.learning_rate / (sqrtf(m_new) + p.eps);
  }
  if (g == 0) {
    WT* w = reinterpret_cast<WT*>(p.dev_weights) + __ldg(p.weights_offsets + t) + row * D;
#pragma unroll
    for (int k = 0; k < kVPL; ++k) {
      const int vv = k * 32 + v;
      if (vv < slice_vecs) {
#pragma unroll
        for (int e = 0; e < kE; e += 4) update_elems4<WT>(w + vv * kE + e, &acc[k][e], mult);
      }
    }
  }
}

struct RunInfo {
  int t;
  int64_t row;
  int D;
  int slice_vecs;
  int gs;
  const char* grad_col;
  bool ok;  // slice is whole, aligned 16-byte vectors and fits the accumulators
};

template <typename KeyT, typename GT>
__device__ __forceinline__ RunInfo describe_run(const BwdDev& p, int64_t s, int max_vpl) {
  RunInfo r;
  const int64_t key = static_cast<int64_t>(reinterpret_cast<const KeyT*>(p.sorted_keys)[s]);
  // table of the key: last t with hash_size_cumsum[t] <= key
  int lo = 0, hi = p.T - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (__ldg(p.hash_size_cumsum + mid) <= key) {
      lo = mid;
    } else {
      hi = mid - 1;
    }
  }
  r.t = lo;
  r.row = key - __ldg(p.hash_size_cumsum + lo);
  const int D_begin = __ldg(p.D_offsets + lo);
  r.D = __ldg(p.D_offsets + lo + 1) - D_begin;
  r.slice_vecs = static_cast<int>((static_cast<int64_t>(r.D) * sizeof(GT)) >> 4);
  r.gs = lanes_per_row(r.slice_vecs);
  r.grad_col = p.grad_output + (p.grad_col_offset + D_begin) * static_cast<int64_t>(sizeof(GT));
  r.ok = ((static_cast<int64_t>(r.D) * sizeof(GT)) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(r.grad_col) & 15) == 0 && r.slice_vecs <= 32 * max_vpl;
  if (!r.ok && p.status != nullptr) atomicOr(p.status, B200TBE_DEV_UNSUPPORTED_SHAPE);
  return r;
}

// ---- streaming reduction of runs -------------------------------------------------------------
// The per-run reduction on the shared-memory ring engine of tbe_stream.cuh: a warp takes up to 31
// consecutive runs, streams the gradient slices of all their lookups through its ring (cp.async,
// two stages in flight), adds them up run by run, and applies the optimizer when the stream crosses
// a run's end. Nothing in the steady state waits on a dependent global load: run starts, keys and
// optimizer state are fetched once per group of runs, the weight rows are prefetched into L2 at
// that point and loaded when their run begins, gradient rows arrive through the ring.

// Applies the optimizer to one row. Lane v holds elements [4v, 4v+4) of vector k*32+v in acc[k].
template <typename WT, int kVPL>
__device__ __forceinline__ void apply_update4(const BwdDev& p, Acc4 (&acc)[kVPL], WT* w_row,
                                              float* m_ptr, int D, int nvec, int lane) {
  float mult = p.learning_rate;
  if (p.optimizer == B200TBE_OPT_ROWWISE_ADAGRAD) {
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < kVPL; ++k) {
      if (k * 32 + lane < nvec) {
        sq = fmaf(acc[k].lo.x, acc[k].lo.x, sq);
        sq = fmaf(acc[k].lo.y, acc[k].lo.y, sq);
        sq = fmaf(acc[k].hi.x, acc[k].hi.x, sq);
        sq = fmaf(acc[k].hi.y, acc[k].hi.y, sq);
      }
    }
    sq = warp_sum(sq);
    float m_new = 0.f;
    if (lane == 0) {
      m_new = *m_ptr + sq / static_cast<float>(D);
      *m_ptr = m_new;
    }
    m_new = __shfl_sync(kFullMask, m_new, 0);
    mult = p.learning_rate / (sqrtf(m_new) + p.eps);
  }
#pragma unroll
  for (int k = 0; k < kVPL; ++k) {
    const int v = k * 32 + lane;
    if (v < nvec) {
      const float g[4] = {acc[k].lo.x, acc[k].lo.y, acc[k].hi.x, acc[k].hi.y};
      update_elems4<WT>(w_row + 4 * v, g, mult);
    }
  }
}

// Weight vector of 4 elements as loaded from global memory, and its update.
template <typename WT>
struct WVec4;
template <>
struct WVec4<float> {
  using Raw = uint4;
  static __device__ __forceinline__ void update_store(float* dst, Raw w, const float (&g)[4], float mult) {
    float4 x = make_float4(__uint_as_float(w.x), __uint_as_float(w.y), __uint_as_float(w.z),
                           __uint_as_float(w.w));
    x.x = fmaf(-mult, g[0], x.x);
    x.y = fmaf(-mult, g[1], x.y);
    x.z = fmaf(-mult, g[2], x.z);
    x.w = fmaf(-mult, g[3], x.w);
    *reinterpret_cast<float4*>(dst) = x;
  }
};
template <>
struct WVec4<__half> {
  using Raw = uint2;
  static __device__ __forceinline__ void update_store(__half* dst, Raw w, const float (&g)[4], float mult) {
    float2 a = half2_bits_to_float2(w.x), b = half2_bits_to_float2(w.y);
    a.x = fmaf(-mult, g[0], a.x);
    a.y = fmaf(-mult, g[1], a.y);
    b.x = fmaf(-mult, g[2], b.x);
    b.y = fmaf(-mult, g[3], b.y);
    // round to nearest even
    *reinterpret_cast<uint2*>(dst) = make_uint2(float2_to_half2_bits(a.x, a.y), float2_to_half2_bits(b.x, b.y));
  }
};

// Optimizer step for one row whose weights (w_regs) and state (m_old, valid on lane 0) were loaded
// earlier. Lane v holds elements [4v, 4v+4) of vector k*32+v in acc[k].
template <typename WT, int kVPL>
__device__ __forceinline__ void apply_update_preloaded(const BwdDev& p, Acc4 (&acc)[kVPL],
                                                       typename WVec4<WT>::Raw (&w_regs)[kVPL],
                                                       float m_old, WT* w_row, float* m_ptr, int D,
                                                       int nvec, int lane) {
  float mult = p.learning_rate;
  if (p.optimizer == B200TBE_OPT_ROWWISE_ADAGRAD) {
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < kVPL; ++k) {
      if (k * 32 + lane < nvec) {
        sq = fmaf(acc[k].lo.x, acc[k].lo.x, sq);
        sq = fmaf(acc[k].lo.y, acc[k].lo.y, sq);
        sq = fmaf(acc[k].hi.x, acc[k].hi.x, sq);
        sq = fmaf(acc[k].hi.y, acc[k].hi.y, sq);
      }
    }
    sq = warp_sum(sq);
    const float m_new = __shfl_sync(kFullMask, m_old, 0) + sq / static_cast<float>(D);
    if (lane == 0) *m_ptr = m_new;
    mult = p.learning_rate / (sqrtf(m_new) + p.eps);
  }
#pragma unroll
  for (int k = 0; k < kVPL; ++k) {
    const int v = k * 32 + lane;
    if (v < nvec) {
      const float g[4] = {acc[k].lo.x, acc[k].lo.y, acc[k].hi.x, acc[k].hi.y};
      WVec4<WT>::update_store(w_row + 4 * v, w_regs[k], g, mult);
    }
  }
}

#include "tbe_backward_sweep.cuh"

struct RunGroup {
  int t;                 // table of every run in the group
  int D;
  int nvec;              // D / 4
  int copy_bytes;        // bytes of a gradient slice
  const char* grad_col;  // grad_output + column of table t, in bytes
  int64_t bag0;          // t * B
};

// Reduces and updates the runs [first_run, first_run + nb) (nb <= 31), which all belong to table
// g.t and are no longer than kLongRun. Lane j holds, for run j: its start (my_start, absolute
// sorted position; lane nb holds the end of the last run) and its row id (my_row).
template <typename KeyT, typename WT, typename GT, int kVPL>
__device__ __forceinline__ void stream_runs(const BwdDev& p, const RunGroup& g, uint32_t my_start,
                                            int64_t my_row, int nb, WarpRing& ring, int lane,
                                            float* partial_dst = nullptr) {
  using Row = FloatRow<GT>;
  const uint32_t p_begin = __shfl_sync(kFullMask, my_start, 0);
  const int my_off = lane <= nb ? static_cast<int>(my_start - p_begin) : 0x7fffffff;
  const int total = __shfl_sync(kFullMask, my_off, nb);
  const int rows_per_stage = min(32, kStageBytes / g.copy_bytes);
  const int num_stages = (total + rows_per_stage - 1) / rows_per_stage;
  const bool weighted = p.per_sample_weights != nullptr;
  const bool mean = p.pooling_mode == B200TBE_POOL_MEAN;
  const bool scaled = weighted || mean;
  const uint32_t* vals = p.sorted_vals + p_begin;

  // this lane's run: where its weights and state live; pull them towards L2 now
  WT* my_w = reinterpret_cast<WT*>(p.dev_weights) + __ldg(p.weights_offsets + g.t) + my_row * g.D;
  float* my_m = p.optimizer == B200TBE_OPT_ROWWISE_ADAGRAD
                    ? p.momentum1 + __ldg(p.momentum1_offsets + g.t) + my_row
                    : nullptr;
  if (lane < nb && partial_dst == nullptr) {
    for (int off = 0; off < g.D * static_cast<int>(sizeof(WT)); off += 128)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(my_w) + off));
    if (my_m != nullptr) asm volatile("prefetch.global.L2 [%0];" ::"l"(my_m));
  }

  Acc4 acc[kVPL];
#pragma unroll
  for (int k = 0; k < kVPL; ++k) acc[k].lo = acc[k].hi = make_float2(0.f, 0.f);
  float bias_unused = 0.f;
  int cur_run = 0;
  int cur_end = __shfl_sync(kFullMask, my_off, 1);

  // weights and state of the run being summed are loaded when the run begins, one run ahead of
  // their use, so the update at the run's end does not wait on them
  typename WVec4<WT>::Raw w_regs[kVPL];
  float m_old = 0.f;
  WT* w_row = nullptr;
  float* m_ptr = nullptr;
  auto load_run_state = [&](int run) {
    w_row = reinterpret_cast<WT*>(__shfl_sync(kFullMask, reinterpret_cast<unsigned long long>(my_w), run));
    m_ptr = reinterpret_cast<float*>(__shfl_sync(kFullMask, reinterpret_cast<unsigned long long>(my_m), run));
#pragma unroll
    for (int k = 0; k < kVPL; ++k) {
      const int v = k * 32 + lane;
      if (v < g.nvec) w_regs[k] = *reinterpret_cast<const typename WVec4<WT>::Raw*>(w_row + 4 * v);
    }
    if (lane == 0 && m_ptr != nullptr) m_old = *m_ptr;
  };
  if (partial_dst == nullptr) load_run_state(0);

  auto flush = [&]() {
    if (partial_dst != nullptr) {
      // a chunk of a long run: its sum goes to scratch, the update happens once all chunks are in
#pragma unroll
      for (int k = 0; k < kVPL; ++k) {
        const int v = k * 32 + lane;
        if (v < g.nvec)
          *reinterpret_cast<float4*>(partial_dst + 4 * v) =
              make_float4(acc[k].lo.x, acc[k].lo.y, acc[k].hi.x, acc[k].hi.y);
      }
    } else {
      apply_update_preloaded<WT, kVPL>(p, acc, w_regs, m_old, w_row, m_ptr, g.D, g.nvec, lane);
    }
#pragma unroll
    for (int k = 0; k < kVPL; ++k) acc[k].lo = acc[k].hi = make_float2(0.f, 0.f);
    ++cur_run;
    cur_end = __shfl_sync(kFullMask, my_off, (cur_run + 1) & 31);
    if (cur_run < nb && partial_dst == nullptr) load_run_state(cur_run);
  };

  const int chunks = g.copy_bytes >> 4;
  const int copy_iters = (rows_per_stage * chunks + 31) >> 5;
  const int lane_row0 = lane / chunks, lane_chunk0 = lane - lane_row0 * chunks;
  const int row_step = 32 / chunks, chunk_step = 32 - row_step * chunks;

  constexpr int kAhead = 3;
  uint32_t val_q[kAhead] = {};
  int issue_pos = lane;
  int issue_slot = 0;
  auto load_val = [&](int pos) -> uint32_t {
    return (lane < rows_per_stage && pos < total) ? __ldg(vals + pos) : kInvalidPayload;
  };
  auto issue = [&]() {
    const int slot = issue_slot;
    const int pos = issue_pos;
    const uint32_t payload = val_q[0];
#pragma unroll
    for (int q = 0; q + 1 < kAhead; ++q) val_q[q] = val_q[q + 1];
    val_q[kAhead - 1] = load_val(pos + kAhead * rows_per_stage);
    issue_pos += rows_per_stage;
    issue_slot = issue_slot + 1 == kStages ? 0 : issue_slot + 1;
    const bool ok = lane < rows_per_stage && pos < total && payload != kInvalidPayload;
    const uint32_t vmask = __ballot_sync(kFullMask, ok);
    const char* my_src = nullptr;
    if (ok) {
      int64_t bag = payload;
      float w = 1.f;
      if (weighted) {
        w = __ldg(p.per_sample_weights + payload);
        bag = __ldg(p.bag_of_pos + payload);
      }
      if (mean) w /= static_cast<float>(bag_length(p, bag));
      if (scaled) ring.weights[slot][lane] = w;
      my_src = g.grad_col + (bag - g.bag0) * p.grad_stride * static_cast<int64_t>(sizeof(GT));
    }
    if (lane == 0) ring.valid[slot] = vmask;
    uint32_t dst = smem_u32(ring.rows[slot]) + (lane << 4);
    int row = lane_row0, chunk = lane_chunk0;
    for (int it = 0; it < copy_iters; ++it) {
      const char* src = reinterpret_cast<const char*>(
          __shfl_sync(kFullMask, reinterpret_cast<unsigned long long>(my_src), row & 31));
      if (row < rows_per_stage && src != nullptr)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src + (chunk << 4))
                     : "memory");
      row += row_step;
      chunk += chunk_step;
      if (chunk >= chunks) {
        chunk -= chunks;
        ++row;
      }
      dst += 512;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

#pragma unroll
  for (int q = 0; q < kAhead; ++q) val_q[q] = load_val(lane + q * rows_per_stage);
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < num_stages) {
      issue();
    } else {
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
  }
  __syncwarp();

  int slot = 0;
  int pos0 = 0;
  for (int stage = 0; stage < num_stages; ++stage) {
    if (stage + kStages - 1 < num_stages) {
      issue();
    } else {
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    __syncwarp();
    asm volatile("cp.async.wait_group %0;" ::"n"(kStages - 1) : "memory");
    __syncwarp();
    const uint32_t vmask = ring.valid[slot];
    const int nr = total - pos0 < rows_per_stage ? total - pos0 : rows_per_stage;
    const uint32_t rows_addr = smem_u32(ring.rows[slot]);
    uint32_t mult_addr = 0;
    if (scaled) {
      ring.mult[slot][lane] = make_float2(((vmask >> lane) & 1u) ? ring.weights[slot][lane] : 0.f, 0.f);
      mult_addr = smem_u32(ring.mult[slot]);
      __syncwarp();
    }
    const bool all_valid = vmask == (nr == 32 ? 0xffffffffu : ((1u << nr) - 1u));
    constexpr int kG = kVPL == 1 ? 4 : (kVPL == 2 ? 2 : 1);
    int r = 0;
    uint32_t row_addr = rows_addr;
    uint32_t m_addr = mult_addr;
    const int m_step = scaled ? 8 : 0;
    while (r < nr) {
      const int left_in_run = cur_end - (pos0 + r);
      if (all_valid && left_in_run >= kG && nr - r >= kG) {
        consume<Row, kVPL, kG>(acc, bias_unused, row_addr, m_addr, g.copy_bytes, g.nvec, lane);
        r += kG;
        row_addr += kG * g.copy_bytes;
        m_addr += kG * m_step;
      } else {
        while (pos0 + r == cur_end) flush();
        if ((vmask >> r) & 1u)
          consume<Row, kVPL, 1>(acc, bias_unused, row_addr, m_addr, g.copy_bytes, g.nvec, lane);
        ++r;
        row_addr += g.copy_bytes;
        m_addr += m_step;
      }
    }
    __syncwarp();
    pos0 += rows_per_stage;
    slot = slot + 1 == kStages ? 0 : slot + 1;
  }
  while (cur_run < nb) flush();
}

// Persistent, one CTA per SM: warps stride over groups of 31 consecutive runs. A group is cut where
// the table changes and around runs longer than kLongRun, which are recorded for the chunked path.
template <typename KeyT, typename WT, typename GT, int kVPL>
__global__ void __launch_bounds__(kStreamThreads, 1)
    reduce_runs_stream_kernel(const __grid_constant__ BwdDev p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  WarpRing* rings = reinterpret_cast<WarpRing*>(smem_raw);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  WarpRing& ring = rings[warp];
  const int64_t runs = p.counters[0];
  const int64_t groups = (runs + 30) / 31;
  const int64_t stride_groups = static_cast<int64_t>(gridDim.x) * kStreamWarps;
  const KeyT* keys = reinterpret_cast<const KeyT*>(p.sorted_keys);
  for (int64_t grp = static_cast<int64_t>(blockIdx.x) * kStreamWarps + warp; grp < groups;
       grp += stride_groups) {
    const int64_t run0 = grp * 31;
    const int n_runs = runs - run0 < 31 ? static_cast<int>(runs - run0) : 31;
    // lane j: start of run j (lane n_runs: end of the last run), its key, table and length
    const uint32_t my_start = lane <= n_runs ? p.run_start[run0 + lane] : 0u;
    const uint32_t next_start = __shfl_down_sync(kFullMask, my_start, 1);
    int my_t = -1;
    int64_t my_row = 0;
    bool my_long = false;
    if (lane < n_runs) {
      const int64_t key = static_cast<int64_t>(keys[my_start]);
      int lo = 0, hi = p.T - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (__ldg(p.hash_size_cumsum + mid) <= key) {
          lo = mid;
        } else {
          hi = mid - 1;
        }
      }
      my_t = lo;
      my_row = key - __ldg(p.hash_size_cumsum + lo);
      my_long = next_start - my_start > static_cast<uint32_t>(kLongRun);
    }
    if (my_long) {
      const uint32_t chunks = (next_start - my_start + kLongRun - 1) / kLongRun;
      const uint32_t slot = atomicAdd(p.counters + 1, 1u);
      const uint32_t chunk0 = atomicAdd(p.counters + 2, chunks);
      p.long_run[slot] = static_cast<uint32_t>(run0 + lane);
      p.long_chunk0[slot] = chunk0;
      for (uint32_t c = 0; c < chunks; ++c) p.chunk_run[chunk0 + c] = slot;
    }
    const uint32_t long_mask = __ballot_sync(kFullMask, my_long);
    const int prev_t = __shfl_up_sync(kFullMask, my_t, 1);
    // a new segment starts at lane 0, after a long run, and where the table changes
    const uint32_t cut_mask = __ballot_sync(
        kFullMask, lane < n_runs && (lane == 0 || my_t != prev_t || ((long_mask >> (lane - 1)) & 1u)));
    int a = 0;
    while (a < n_runs) {
      if ((long_mask >> a) & 1u) {
        ++a;
        continue;
      }
      // segment [a, b): up to the next cut or long run
      const uint32_t later = (cut_mask | long_mask) & ~((2u << a) - 1u);
      int b = later ? __ffs(later) - 1 : n_runs;
      if (b > n_runs) b = n_runs;
      RunGroup g;
      g.t = __shfl_sync(kFullMask, my_t, a);
      const int D_begin = __ldg(p.D_offsets + g.t);
      g.D = __ldg(p.D_offsets + g.t + 1) - D_begin;
      g.nvec = g.D >> 2;
      g.copy_bytes = g.D * static_cast<int>(sizeof(GT));
      g.grad_col = p.grad_output + (p.grad_col_offset + D_begin) * static_cast<int64_t>(sizeof(GT));
      g.bag0 = static_cast<int64_t>(g.t) * p.B;
      const bool ok = (g.copy_bytes & 15) == 0 && (reinterpret_cast<uintptr_t>(g.grad_col) & 15) == 0 &&
                      g.nvec <= 32 * kVPL && g.copy_bytes <= kStageBytes && g.D > 0;
      if (ok) {
        // re-base the lanes so that lane j describes run a + j
        const uint32_t seg_start = __shfl_sync(kFullMask, my_start, (lane + a) & 31);
        const int64_t seg_row = __shfl_sync(kFullMask, my_row, (lane + a) & 31);
        stream_runs<KeyT, WT, GT, kVPL>(p, g, seg_start, seg_row, b - a, ring, lane);
      } else if (lane == 0 && p.status != nullptr) {
        atomicOr(p.status, B200TBE_DEV_UNSUPPORTED_SHAPE);
      }
      a = b;
    }
  }
}

// Persistent, one CTA per SM: one warp per chunk of a long run, streamed through the ring like a
// short run; the chunk's sum goes to scratch.
template <typename KeyT, typename WT, typename GT, int kVPL>
__global__ void __launch_bounds__(kStreamThreads, 1)
    reduce_chunks_stream_kernel(const __grid_constant__ BwdDev p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  WarpRing* rings = reinterpret_cast<WarpRing*>(smem_raw);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  WarpRing& ring = rings[warp];
  const int64_t chunks = p.counters[2];
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kStreamWarps;
  const KeyT* keys = reinterpret_cast<const KeyT*>(p.sorted_keys);
  for (int64_t c = static_cast<int64_t>(blockIdx.x) * kStreamWarps + warp; c < chunks; c += stride) {
    const uint32_t slot = p.chunk_run[c];
    const uint32_t run = p.long_run[slot];
    const int64_t first = p.long_chunk0[slot];
    const uint32_t s_run = p.run_start[run], e_run = p.run_start[run + 1];
    const uint32_t s = s_run + static_cast<uint32_t>(c - first) * kLongRun;
    const uint32_t e = s + kLongRun < e_run ? s + kLongRun : e_run;
    const int64_t key = static_cast<int64_t>(keys[s_run]);
    int lo = 0, hi = p.T - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (__ldg(p.hash_size_cumsum + mid) <= key) {
        lo = mid;
      } else {
        hi = mid - 1;
      }
    }
    RunGroup g;
    g.t = lo;
    const int D_begin = __ldg(p.D_offsets + g.t);
    g.D = __ldg(p.D_offsets + g.t + 1) - D_begin;
    g.nvec = g.D >> 2;
    g.copy_bytes = g.D * static_cast<int>(sizeof(GT));
    g.grad_col = p.grad_output + (p.grad_col_offset + D_begin) * static_cast<int64_t>(sizeof(GT));
    g.bag0 = static_cast<int64_t>(g.t) * p.B;
    const bool ok = (g.copy_bytes & 15) == 0 && (reinterpret_cast<uintptr_t>(g.grad_col) & 15) == 0 &&
                    g.nvec <= 32 * kVPL && g.copy_bytes <= kStageBytes && g.D > 0;
    if (!ok) continue;  // flagged by the kernel that recorded the run
    const uint32_t my_start = lane == 0 ? s : e;
    stream_runs<KeyT, WT, GT, kVPL>(p, g, my_start, 0, 1, ring, lane, p.partials + c * p.max_D);
  }
}

// Persistent: one warp per long run adds the run's partial rows in chunk order and updates.
template <typename KeyT, typename WT, typename GT, int kVPL>
__global__ void __launch_bounds__(kBwdThreads) finish_long_runs_kernel(BwdDev p) {
  constexpr int kE = RowVec<GT>::kElems;
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = static_cast<int64_t>(blockIdx.x) * kBwdWarps + (threadIdx.x >> 5);
  const int64_t num_warps = static_cast<int64_t>(gridDim.x) * kBwdWarps;
  const int64_t long_runs = p.counters[1];
  for (int64_t i = warp0; i < long_runs; i += num_warps) {
    const uint32_t run = p.long_run[i];
    const int64_t s = p.run_start[run], e = p.run_start[run + 1];
    const int64_t chunks = (e - s + kLongRun - 1) / kLongRun;
    const RunInfo r = describe_run<KeyT, GT>(p, s, kVPL);
    if (!r.ok) continue;
    const int g = lane / r.gs, v = lane - g * r.gs;
    float acc[kVPL][kE];
#pragma unroll
    for (int k = 0; k < kVPL; ++k)
#pragma unroll
      for (int j = 0; j < kE; ++j) acc[k][j] = 0.f;
    if (g == 0) {
      const float* src = p.partials + static_cast<int64_t>(p.long_chunk0[i]) * p.max_D;
      for (int64_t c = 0; c < chunks; ++c, src += p.max_D) {
#pragma unroll
        for (int k = 0; k < kVPL; ++k) {
          const int vv = k * 32 + v;
          if (vv < r.slice_vecs) {
#pragma unroll
            for (int j = 0; j < kE; j += 4) {
              const float4 x = *reinterpret_cast<const float4*>(src + vv * kE + j);
              acc[k][j] += x.x;
              acc[k][j + 1] += x.y;
              acc[k][j + 2] += x.z;
              acc[k][j + 3] += x.w;
            }
          }
        }
      }
    }
    apply_update<WT, kE, kVPL>(p, acc, r.t, r.row, r.D, r.gs, r.slice_vecs, lane);
  }
}

size_t align256(size_t x) { return (x + 255) & ~size_t{255}; }

// Rows of up to kSweepMaxD elements take the sweep path, wider ones the ring engine.
constexpr int kSweepMaxD = 512;
constexpr int kRingMaxD = 1024;

struct ScratchLayout {
  size_t keys_a, keys_b, vals_a, vals_b, bag_of_pos, run_start, tile_heads, counters, long_run,
      long_chunk0, chunk_run, partials, sort, plan, span_flags, total;
  int key_bytes;
  bool sweep;
  int64_t max_long, max_chunks, max_tiles;
};

ScratchLayout layout_for(int64_t n, int bits, int max_D, int T) {
  ScratchLayout L{};
  L.sweep = max_D <= kSweepMaxD;
  L.key_bytes = (L.sweep || bits <= 32) ? 4 : 8;
  const size_t nn = static_cast<size_t>(n > 0 ? n : 1);
  const size_t row = static_cast<size_t>(max_D > 0 ? max_D : 1) * 4;
  size_t at = 0;
  auto take = [&](size_t bytes) {
    const size_t here = at;
    at += align256(bytes);
    return here;
  };
  L.keys_a = take(nn * L.key_bytes);
  L.keys_b = take(nn * L.key_bytes);
  L.vals_a = take(nn * 4);
  L.vals_b = take(nn * 4);
  L.bag_of_pos = take(nn * 4);
  L.counters = take(256);
  if (L.sweep) {
    // every table's last tile may be partial
    L.max_tiles = sort_plan_max_tiles(n, T);
    L.plan = take(sort_plan_bytes(n, T));
    L.span_flags = take(static_cast<size_t>(L.max_tiles) * kSpansPerTile * 4);
    L.partials = take(static_cast<size_t>(L.max_tiles) * kSpansPerTile * 2 * row);
    L.sort = take(radix_sort_planned_scratch_bytes(L.max_tiles));
  } else {
    L.max_long = n / kLongRun + 1;
    L.max_chunks = 2 * (n / kLongRun) + 2;
    L.run_start = take((nn + 1) * 4);
    L.tile_heads = take(static_cast<size_t>((n + kSegTile - 1) / kSegTile + 1) * 4);
    L.long_run = take(static_cast<size_t>(L.max_long) * 4);
    L.long_chunk0 = take(static_cast<size_t>(L.max_long) * 4);
    L.chunk_run = take(static_cast<size_t>(L.max_chunks) * 4);
    L.partials = take(static_cast<size_t>(L.max_chunks) * row);
    L.sort = take(radix_sort_scratch_bytes(n));
  }
  L.total = at;
  return L;
}

int persistent_grid() {
  // one wave of CTAs that all fit at once: 148 SMs x a few CTAs each
  return kNumSMs * 6;
}

// ---- wide rows: ring engine ---------------------------------------------------------------------
template <typename KeyT, typename WT, typename GT, int kVPL>
int run_reduce(const BwdDev& d, cudaStream_t stream) {
  const int grid = persistent_grid();
  auto stream_kernel = reduce_runs_stream_kernel<KeyT, WT, GT, kVPL>;
  if (cudaFuncSetAttribute(stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kStreamSmemBytes)) != cudaSuccess)
    return B200TBE_ERR_LAUNCH;
  stream_kernel<<<kNumSMs, kStreamThreads, kStreamSmemBytes, stream>>>(d);
  auto chunk_kernel = reduce_chunks_stream_kernel<KeyT, WT, GT, kVPL>;
  if (cudaFuncSetAttribute(chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kStreamSmemBytes)) != cudaSuccess)
    return B200TBE_ERR_LAUNCH;
  chunk_kernel<<<kNumSMs, kStreamThreads, kStreamSmemBytes, stream>>>(d);
  finish_long_runs_kernel<KeyT, WT, GT, kVPL><<<grid, kBwdThreads, 0, stream>>>(d);
  return launch_status();
}

template <typename KeyT, typename IndexT>
int run_backward_wide(BwdDev d, const b200tbe_backward_params* p, const ScratchLayout& L, char* scratch,
                      cudaStream_t stream) {
  const int64_t n = p->num_indices;
  KeyT* keys_a = reinterpret_cast<KeyT*>(scratch + L.keys_a);
  KeyT* keys_b = reinterpret_cast<KeyT*>(scratch + L.keys_b);
  uint32_t* vals_a = reinterpret_cast<uint32_t*>(scratch + L.vals_a);
  uint32_t* vals_b = reinterpret_cast<uint32_t*>(scratch + L.vals_b);
  uint32_t* tile_heads = reinterpret_cast<uint32_t*>(scratch + L.tile_heads);
  const bool weighted = p->per_sample_weights != nullptr;

  if (cudaMemsetAsync(d.counters, 0, 256, stream) != cudaSuccess) return B200TBE_ERR_LAUNCH;
  const int64_t bags = static_cast<int64_t>(p->T) * p->B;
  const int64_t lin_ctas = (bags + 32 * kBwdWarps - 1) / (32 * kBwdWarps);
  if (lin_ctas > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  if (weighted) {
    linearize_kernel<KeyT, IndexT, true>
        <<<static_cast<unsigned>(lin_ctas), kBwdThreads, 0, stream>>>(d, keys_a, vals_a);
  } else {
    linearize_kernel<KeyT, IndexT, false>
        <<<static_cast<unsigned>(lin_ctas), kBwdThreads, 0, stream>>>(d, keys_a, vals_a);
  }
  bool in_b = false;
  int st = radix_sort_pairs(keys_a, vals_a, keys_b, vals_b, n, sizeof(KeyT),
                            p->total_hash_size_bits, scratch + L.sort,
                            radix_sort_scratch_bytes(n), &in_b, stream);
  if (st != B200TBE_OK) return st;
  const KeyT* keys = in_b ? keys_b : keys_a;
  d.sorted_keys = keys;
  d.sorted_vals = in_b ? vals_b : vals_a;

  const int64_t seg_tiles = (n + kSegTile - 1) / kSegTile;
  count_heads_kernel<KeyT><<<static_cast<unsigned>(seg_tiles), kSegThreads, 0, stream>>>(keys, n, tile_heads);
  scan_single_cta_kernel<<<1, kScanThreads, 0, stream>>>(tile_heads, seg_tiles, d.counters);
  write_run_starts_kernel<KeyT><<<static_cast<unsigned>(seg_tiles), kSegThreads, 0, stream>>>(
      keys, n, tile_heads, d.counters, d.run_start);

  // everything above needed only the indices; the gradients are read from here on
  if (p->grad_ready_event != nullptr &&
      cudaStreamWaitEvent(stream, static_cast<cudaEvent_t>(p->grad_ready_event), 0) != cudaSuccess)
    return B200TBE_ERR_LAUNCH;
  // a lane of the ring engine holds kVPL vectors of 4 ELEMENTS, whatever the gradient type:
  // 1024 elements need 8
  const bool w32 = p->weights_dtype == B200TBE_FP32, g32 = p->grad_dtype == B200TBE_FP32;
  if (w32 && g32) return run_reduce<KeyT, float, float, 8>(d, stream);
  if (!w32 && g32) return run_reduce<KeyT, __half, float, 8>(d, stream);
  if (w32 && !g32) return run_reduce<KeyT, float, __half, 8>(d, stream);
  return run_reduce<KeyT, __half, __half, 8>(d, stream);
}

// ---- rows of up to 512 elements: plan, segmented sort, sweep --------------------------------------
template <typename WT, typename GT, bool kScaled, int GS, int kC>
int launch_sweep(const BwdDev& d, int max_tiles, cudaStream_t stream) {
  constexpr int kSpansPerCta = kSweepWarps * (32 / GS);
  const int64_t ctas = static_cast<int64_t>(max_tiles) * (kSpansPerTile / kSpansPerCta);
  const int64_t spans = static_cast<int64_t>(max_tiles) * kSpansPerTile;
  if (ctas > 0x7fffffff || spans / kFinishWarps > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  sweep_runs_kernel<WT, GT, kScaled, GS, kC, sweep_ctas_per_sm<WT, GT, kC>()>
      <<<static_cast<unsigned>(ctas), kSweepThreads, 0, stream>>>(d);
  finish_open_runs_kernel<WT, GS, kC>
      <<<static_cast<unsigned>(spans / kFinishWarps), kFinishWarps * 32, 0, stream>>>(d);
  return launch_status();
}

template <typename WT, typename GT, bool kScaled>
int dispatch_sweep_shape(const BwdDev& d, int max_tiles, cudaStream_t stream) {
  // lanes per row x quads per lane: rows of up to 128 elements get one quad per lane of the
  // smallest group that holds them, wider rows the whole warp with several quads per lane
  if (d.max_D <= 32) return launch_sweep<WT, GT, kScaled, 8, 1>(d, max_tiles, stream);
  if (d.max_D <= 64) return launch_sweep<WT, GT, kScaled, 16, 1>(d, max_tiles, stream);
  if (d.max_D <= 128) return launch_sweep<WT, GT, kScaled, 32, 1>(d, max_tiles, stream);
  if (d.max_D <= 256) return launch_sweep<WT, GT, kScaled, 32, 2>(d, max_tiles, stream);
  return launch_sweep<WT, GT, kScaled, 32, 4>(d, max_tiles, stream);
}

template <typename WT, typename GT>
int dispatch_sweep_scaled(const BwdDev& d, int max_tiles, cudaStream_t stream) {
  if (d.per_sample_weights != nullptr || d.pooling_mode == B200TBE_POOL_MEAN)
    return dispatch_sweep_shape<WT, GT, true>(d, max_tiles, stream);
  return dispatch_sweep_shape<WT, GT, false>(d, max_tiles, stream);
}

int ceil_log2(int64_t x) {
  int b = 0;
  while (b < 62 && (int64_t{1} << b) < x) ++b;
  return b;
}

template <typename IndexT>
int run_backward_sweep(BwdDev d, const b200tbe_backward_params* p, const ScratchLayout& L, char* scratch,
                       cudaStream_t stream) {
  const int64_t n = p->num_indices;
  uint32_t* keys_a = reinterpret_cast<uint32_t*>(scratch + L.keys_a);
  uint32_t* keys_b = reinterpret_cast<uint32_t*>(scratch + L.keys_b);
  uint32_t* vals_a = reinterpret_cast<uint32_t*>(scratch + L.vals_a);
  uint32_t* vals_b = reinterpret_cast<uint32_t*>(scratch + L.vals_b);
  const int max_tiles = static_cast<int>(L.max_tiles);
  const bool weighted = p->per_sample_weights != nullptr;

  // bits that differ inside a table: those of the largest table's last row id
  int key_bits = p->total_hash_size_bits < 32 ? p->total_hash_size_bits : 32;
  if (p->max_table_rows > 0 && ceil_log2(p->max_table_rows) < key_bits) key_bits = ceil_log2(p->max_table_rows);
  if (key_bits < 1) key_bits = 1;

  // the lookups of table t are positions [offsets[t * B], offsets[(t + 1) * B])
  SortPlan plan{};
  const uint32_t* seg_start = nullptr;
  int st = build_sort_plan(p->offsets, p->index_bytes, p->T, p->B, n, scratch + L.plan, p->status, &plan,
                           &seg_start, stream);
  if (st != B200TBE_OK) return st;
  const int64_t bags = static_cast<int64_t>(p->T) * p->B;
  const int64_t lin_ctas = (bags + 32 * kBwdWarps - 1) / (32 * kBwdWarps);
  if (lin_ctas > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  if (weighted) {
    linearize_rows_kernel<IndexT, true>
        <<<static_cast<unsigned>(lin_ctas), kBwdThreads, 0, stream>>>(d, key_bits, keys_a, vals_a);
  } else {
    linearize_rows_kernel<IndexT, false>
        <<<static_cast<unsigned>(lin_ctas), kBwdThreads, 0, stream>>>(d, key_bits, keys_a, vals_a);
  }
  bool in_b = false;
  st = radix_sort_pairs_planned(keys_a, vals_a, keys_b, vals_b, n, key_bits, kSweepSortDigitBits,
                                          plan, scratch + L.sort, radix_sort_planned_scratch_bytes(max_tiles),
                                          &in_b, stream);
  if (st != B200TBE_OK) return st;
  d.sorted_keys = in_b ? keys_b : keys_a;
  d.sorted_vals = in_b ? vals_b : vals_a;
  d.seg_start = seg_start;
  d.seg_tile_base = plan.seg_tile_base;
  d.total_tiles = plan.total_tiles;
  d.tile_desc = plan.tile_desc;
  d.span_flags = reinterpret_cast<uint32_t*>(scratch + L.span_flags);

  // everything above needed only the indices; the gradients are read from here on
  if (p->grad_ready_event != nullptr &&
      cudaStreamWaitEvent(stream, static_cast<cudaEvent_t>(p->grad_ready_event), 0) != cudaSuccess)
    return B200TBE_ERR_LAUNCH;
  const bool w32 = p->weights_dtype == B200TBE_FP32, g32 = p->grad_dtype == B200TBE_FP32;
  if (w32 && g32) return dispatch_sweep_scaled<float, float>(d, max_tiles, stream);
  if (!w32 && g32) return dispatch_sweep_scaled<__half, float>(d, max_tiles, stream);
  if (w32 && !g32) return dispatch_sweep_scaled<float, __half>(d, max_tiles, stream);
  return dispatch_sweep_scaled<__half, __half>(d, max_tiles, stream);
}

}  // namespace
}  // namespace b200tbe

using namespace b200tbe;

extern "C" size_t b200tbe_backward_scratch_bytes(int64_t num_indices, int32_t total_hash_size_bits,
                                                 int32_t max_D, int32_t T) {
  if (num_indices < 0 || T < 0) return 0;
  return layout_for(num_indices, total_hash_size_bits, max_D, T).total;
}

extern "C" int b200tbe_backward(const b200tbe_backward_params* p, b200tbe_stream_t stream_) {
  if (p == nullptr) return B200TBE_ERR_BAD_ARG;
  if (p->T < 0 || p->B < 0 || p->max_D < 0 || p->num_indices < 0 || p->max_table_rows < 0)
    return B200TBE_ERR_BAD_ARG;
  if (p->T == 0 || p->B == 0 || p->num_indices == 0) return B200TBE_OK;
  if (p->dev_weights == nullptr || p->weights_offsets == nullptr || p->D_offsets == nullptr ||
      p->hash_size_cumsum == nullptr || p->indices == nullptr || p->offsets == nullptr ||
      p->grad_output == nullptr)
    return B200TBE_ERR_BAD_ARG;
  if (p->index_bytes != 4 && p->index_bytes != 8) return B200TBE_ERR_BAD_ARG;
  if (p->optimizer != B200TBE_OPT_SGD && p->optimizer != B200TBE_OPT_ROWWISE_ADAGRAD)
    return B200TBE_ERR_UNSUPPORTED;
  if (p->optimizer == B200TBE_OPT_ROWWISE_ADAGRAD &&
      (p->momentum1 == nullptr || p->momentum1_offsets == nullptr))
    return B200TBE_ERR_BAD_ARG;
  if (p->pooling_mode != B200TBE_POOL_SUM && p->pooling_mode != B200TBE_POOL_MEAN)
    return B200TBE_ERR_UNSUPPORTED;
  if ((p->weights_dtype != B200TBE_FP32 && p->weights_dtype != B200TBE_FP16) ||
      (p->grad_dtype != B200TBE_FP32 && p->grad_dtype != B200TBE_FP16))
    return B200TBE_ERR_UNSUPPORTED;
  if (p->total_hash_size_bits < 1 || p->total_hash_size_bits > 40) return B200TBE_ERR_UNSUPPORTED;
  if (p->num_indices >= (int64_t{1} << 31)) return B200TBE_ERR_TOO_LARGE;
  if (static_cast<int64_t>(p->T) * p->B >= (int64_t{1} << 32) - 1) return B200TBE_ERR_TOO_LARGE;
  if (p->max_D % 4 != 0 || p->max_D > kRingMaxD) return B200TBE_ERR_UNSUPPORTED;
  const int grad_bytes = p->grad_dtype == B200TBE_FP32 ? 4 : 2;
  // gradient slices are read as whole 16-byte vectors
  if ((p->grad_stride * grad_bytes) % 16 != 0 || (p->grad_col_offset * grad_bytes) % 16 != 0 ||
      !aligned_to(p->grad_output, 16) || !aligned_to(p->dev_weights, 16))
    return B200TBE_ERR_UNSUPPORTED;
  if (p->max_D > kSweepMaxD && (p->max_D * grad_bytes) % 16 != 0) return B200TBE_ERR_UNSUPPORTED;
  // offsets of gradient slices inside one table's columns travel as 32-bit counts of 16 bytes
  if (static_cast<int64_t>(p->B) * p->grad_stride * grad_bytes / 16 >= (int64_t{1} << 32) - 1)
    return B200TBE_ERR_TOO_LARGE;
  const ScratchLayout L = layout_for(p->num_indices, p->total_hash_size_bits, p->max_D, p->T);
  if (p->scratch == nullptr || p->scratch_bytes < L.total || !aligned_to(p->scratch, 256))
    return B200TBE_ERR_SCRATCH;
  char* scratch = static_cast<char*>(p->scratch);

  BwdDev d{};
  d.dev_weights = static_cast<char*>(p->dev_weights);
  d.weights_offsets = p->weights_offsets;
  d.D_offsets = p->D_offsets;
  d.hash_size_cumsum = p->hash_size_cumsum;
  d.indices = p->indices;
  d.offsets = p->offsets;
  d.per_sample_weights = p->per_sample_weights;
  d.grad_output = static_cast<const char*>(p->grad_output);
  d.grad_stride = p->grad_stride;
  d.grad_col_offset = p->grad_col_offset;
  d.momentum1 = p->momentum1;
  d.momentum1_offsets = p->momentum1_offsets;
  d.num_indices = p->num_indices;
  d.T = p->T;
  d.B = p->B;
  d.pooling_mode = p->pooling_mode;
  d.optimizer = p->optimizer;
  d.index_bytes = p->index_bytes;
  d.learning_rate = p->learning_rate;
  d.eps = p->eps;
  d.status = p->status;
  d.bag_of_pos = reinterpret_cast<uint32_t*>(scratch + L.bag_of_pos);
  d.counters = reinterpret_cast<uint32_t*>(scratch + L.counters);
  d.partials = reinterpret_cast<float*>(scratch + L.partials);
  d.max_D = p->max_D;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const bool i64 = p->index_bytes == 8;
  if (L.sweep)
    return i64 ? run_backward_sweep<int64_t>(d, p, L, scratch, stream)
               : run_backward_sweep<int32_t>(d, p, L, scratch, stream);
  d.run_start = reinterpret_cast<uint32_t*>(scratch + L.run_start);
  d.long_run = reinterpret_cast<uint32_t*>(scratch + L.long_run);
  d.long_chunk0 = reinterpret_cast<uint32_t*>(scratch + L.long_chunk0);
  d.chunk_run = reinterpret_cast<uint32_t*>(scratch + L.chunk_run);
  if (L.key_bytes == 4) {
    return i64 ? run_backward_wide<uint32_t, int64_t>(d, p, L, scratch, stream)
               : run_backward_wide<uint32_t, int32_t>(d, p, L, scratch, stream);
  }
  return i64 ? run_backward_wide<unsigned long long, int64_t>(d, p, L, scratch, stream)
             : run_backward_wide<unsigned long long, int32_t>(d, p, L, scratch, stream);
}
