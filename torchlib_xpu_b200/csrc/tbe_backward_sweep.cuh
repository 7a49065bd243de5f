// Backward for rows of at most 512 elements: plan, sweep, finish.
//
// After the segmented sort the lookups of table t occupy sorted positions [seg_start[t],
// seg_start[t+1]) ordered by row, and equal rows are adjacent (a "run"). The reduction is organised
// by LOOKUP, not by run, because a recommender id stream mixes millions of one-lookup runs with
// runs of a hundred thousand lookups:
//   * every tile of the sort plan (4096 sorted positions of one table) is cut into 16 spans of 256
//     positions; a group of GS lanes sweeps one span from left to right, each lane holding kC quads
//     of 4 elements of the running sum (quad c of lane l = elements (c * GS + l) * 4 ...), so one
//     load instruction of a group reads contiguous bytes of one gradient slice. A warp carries
//     32 / GS groups, i.e. that many consecutive spans, through one instruction stream;
//   * per batch of GS positions, lane l fetches position l's row id, its successor's (run end?),
//     and the bag id, turns the bag id into the offset of the gradient slice, and asks L2 for the
//     weight row of every run that ends in the batch -- one batch ahead of its use;
//   * per position: the slice offset arrives by shuffle, four positions' loads are issued before the
//     first is added, and where a run ends the row is updated once, in place ("exact" update);
//   * three rows in four are looked up once. Where a warp carries several groups, updating such a
//     run inside the sweep would run the whole update sequence for one group while the others
//     idle, so the batch's one-lookup runs are left out of the sweep and updated in a pass of their
//     own, one per GROUP and step whichever span they lie in. Rows of 128 elements and more take the
//     whole warp (one group), where every update is full width anyway;
//   * a run that crosses a span boundary leaves partial sums in scratch instead (the piece that
//     ends a run begun earlier -> "head" slot of the span, the piece that begins a run finished
//     later -> "tail" slot); finish_open_runs_kernel adds a run's pieces in span order and updates.
// Nothing depends on scheduling: the order of additions is fixed by the sorted order alone.
//
// Part of tbe_backward.cu: included there inside its namespace, after BwdDev and bag_length.
#pragma once

constexpr int kSpan = 256;                                  // sorted positions per span
constexpr int kSpansPerTile = kSortPlanTile / kSpan;        // 16
// One warp per CTA: spans finish at very different times (a span inside a long run is pure
// streaming, a span of one-lookup runs updates a row every other position), and a CTA keeps its
// slot until its slowest warp is done. Measured on the bench step: 4 warps per CTA 9.65 ms for the
// backward, 2 warps 9.67, 1 warp 8.85 at the same registers, 7.99 with 32 such CTAs per SM.
constexpr int kSweepWarps = 1;
constexpr int kSweepThreads = kSweepWarps * 32;
constexpr int kFinishWarps = 4;
// positions whose gradient slices are in flight per group (fewer when a lane holds more of a row)
template <int kC>
__host__ __device__ constexpr int sweep_loads() {
  return kC <= 2 ? 4 : 2;
}
// one fp16 quad per lane of gradient and of weights costs two registers each per position: eight
// positions in flight where the whole warp sweeps one span; anything wider, or several spans per
// warp (which also keep the one-lookup runs' pass in registers), four (or two)
template <typename WT, typename GT, bool kScaled, int kC, int GS = 32>
__host__ __device__ constexpr int sweep_loads_for() {
  return kC == 1 && GS == 32 && sizeof(GT) == 2 && sizeof(WT) == 2 && !kScaled ? 8 : sweep_loads<kC>();
}
template <typename WT, typename GT, int kC>
__host__ __device__ constexpr int sweep_ctas_per_sm() {
  // CTAs (= warps) per SM; the register file allows 65536 / (32 * this) registers per thread. One quad
  // per lane of fp16 weights fits 64 registers with either gradient type (26 tables x 1 M rows with
  // fp32 gradients: 0.762 ms at 32 CTAs, 0.785 at 24, 0.790 at 28; eight positions in flight at 20 or
  // 16 CTAs: 0.815, 0.854)
  return kC > 2 ? 16 : (kC == 2 ? (sizeof(WT) == 2 && sizeof(GT) == 2 ? 20 : 16) : (sizeof(WT) == 2 ? 32 : 24));
}
constexpr uint32_t kNoSlice = 0xffffffffu;
constexpr uint32_t kSpanTailOwner = 1u;   // the span's last run continues to the right; its piece is in the tail slot
constexpr uint32_t kSpanThrough = 2u;     // the whole span is the middle of one run; its piece is in the head slot

// Four consecutive elements of a row.
template <typename T>
struct Quad;

template <>
struct Quad<float> {
  using Raw = uint4;
  static __device__ __forceinline__ Raw zero() { return make_uint4(0u, 0u, 0u, 0u); }
  static __device__ __forceinline__ Raw load_ro(const char* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
  static __device__ __forceinline__ Raw load(const char* p) { return *reinterpret_cast<const uint4*>(p); }
  static __device__ __forceinline__ float4 to(Raw r) {
    return make_float4(__uint_as_float(r.x), __uint_as_float(r.y), __uint_as_float(r.z),
                       __uint_as_float(r.w));
  }
  static __device__ __forceinline__ void add(float4& a, Raw r) {
    a.x += __uint_as_float(r.x);
    a.y += __uint_as_float(r.y);
    a.z += __uint_as_float(r.z);
    a.w += __uint_as_float(r.w);
  }
  static __device__ __forceinline__ void store(char* p, float4 f) { *reinterpret_cast<float4*>(p) = f; }
};

template <>
struct Quad<__half> {
  using Raw = uint2;
  static __device__ __forceinline__ Raw zero() { return make_uint2(0u, 0u); }
  static __device__ __forceinline__ Raw load_ro(const char* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }
  static __device__ __forceinline__ Raw load(const char* p) { return *reinterpret_cast<const uint2*>(p); }
  static __device__ __forceinline__ float4 to(Raw r) {
    const float2 a = half2_bits_to_float2(r.x), b = half2_bits_to_float2(r.y);
    return make_float4(a.x, a.y, b.x, b.y);
  }
  // fp16 elements go straight into the fp32 sums (mixed-precision add of sm_100)
  static __device__ __forceinline__ void add(float4& a, Raw r) {
    add_half2(a.x, a.y, r.x);
    add_half2(a.z, a.w, r.y);
  }
  // round to nearest even
  static __device__ __forceinline__ void store(char* p, float4 f) {
    *reinterpret_cast<uint2*>(p) = make_uint2(float2_to_half2_bits(f.x, f.y), float2_to_half2_bits(f.z, f.w));
  }
};

__device__ __forceinline__ float sqrt_fast(float x) {
  float r;
  asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// ---- linearize with per-table keys -------------------------------------------------------------
// As linearize_kernel, but the key is the row id alone: the table is implied by the position.
template <typename IndexT, bool kWeighted>
__global__ void __launch_bounds__(kBwdThreads)
    linearize_rows_kernel(BwdDev p, int key_bits, uint32_t* __restrict__ keys, uint32_t* __restrict__ vals) {
  const int lane = threadIdx.x & 31;
  const int64_t total_bags = static_cast<int64_t>(p.T) * p.B;
  const int64_t bag0 = (static_cast<int64_t>(blockIdx.x) * kBwdWarps + (threadIdx.x >> 5)) * 32;
  if (bag0 >= total_bags) return;
  const int nb = total_bags - bag0 < 32 ? static_cast<int>(total_bags - bag0) : 32;
  const int64_t begin = load_index<IndexT>(p.offsets, bag0);
  int64_t end = load_index<IndexT>(p.offsets, bag0 + nb);
  if (end > p.num_indices) end = p.num_indices;
  const int64_t mine = load_index<IndexT>(p.offsets, bag0 + (lane < nb ? lane : nb));
  const uint32_t my_start = static_cast<uint32_t>(mine - begin);
  const int my_t = static_cast<int>((bag0 + (lane < nb ? lane : nb - 1)) / p.B);
  int64_t my_rows = __ldg(p.hash_size_cumsum + my_t + 1) - __ldg(p.hash_size_cumsum + my_t);
  const int64_t sortable = int64_t{1} << key_bits;
  if (my_rows > sortable) {   // the caller's bound on rows per table was too small for this table
    if (p.status != nullptr) atomicOr(p.status, B200TBE_DEV_UNSUPPORTED_SHAPE);
    my_rows = sortable;
  }
  const uint32_t total = end > begin ? static_cast<uint32_t>(end - begin) : 0u;
  // four batches of 32 ids are requested before the first is turned into a key
  constexpr int kBatches = 4;
  for (uint32_t base = 0; base < total; base += 32 * kBatches) {
    int64_t ids[kBatches];
#pragma unroll
    for (int k = 0; k < kBatches; ++k) {
      const uint32_t rel = base + 32 * k + lane;
      ids[k] = rel < total ? load_index<IndexT>(p.indices, begin + rel) : 0;
    }
#pragma unroll
    for (int k = 0; k < kBatches; ++k) {
      const uint32_t rel = base + 32 * k + lane;
      int b = 0;
#pragma unroll
      for (int step = 16; step > 0; step >>= 1) {
        const int cand = b + step;
        const uint32_t s = __shfl_sync(kFullMask, my_start, cand & 31);
        if (cand < nb && s <= rel) b = cand;
      }
      const int64_t rows = __shfl_sync(kFullMask, my_rows, b);
      if (rel < total) {
        const int64_t j = begin + rel;
        int64_t idx = ids[k];
        const uint32_t bag = static_cast<uint32_t>(bag0 + b);
        uint32_t payload = kWeighted ? static_cast<uint32_t>(j) : bag;
        if (idx < 0 || idx >= rows) {
          if (p.status != nullptr) atomicOr(p.status, B200TBE_DEV_INDEX_OUT_OF_RANGE);
          idx = 0;
          payload = kInvalidPayload;
        }
        keys[j] = static_cast<uint32_t>(idx);
        vals[j] = payload;
        if (kWeighted) p.bag_of_pos[j] = bag;
      }
    }
  }
}

// ---- sweep ----------------------------------------------------------------------------------------
// What a span's table looks like (the same for every group of a warp: a tile lies in one table).
template <typename WT, typename GT>
struct SweepTable {
  int D;
  char* w_lane;          // row 0 of the table at this lane's first quad
  float* mbase;          // row-wise optimizer state of row 0, or null
  const char* g_lane;    // gradient columns of the table in sample 0, at this lane's first quad
  uint32_t bag0;         // t * B
  int64_t gstride_bytes;
  int row_bytes;         // D * sizeof(WT)
  bool ok;
};

template <typename WT, typename GT, int GS, int kC>
__device__ __forceinline__ SweepTable<WT, GT> sweep_table(const BwdDev& p, int t, int gl) {
  SweepTable<WT, GT> s;
  const int D_begin = __ldg(p.D_offsets + t);
  s.D = __ldg(p.D_offsets + t + 1) - D_begin;
  char* w0 = p.dev_weights + __ldg(p.weights_offsets + t) * static_cast<int64_t>(sizeof(WT));
  const char* g0 = p.grad_output + (p.grad_col_offset + D_begin) * static_cast<int64_t>(sizeof(GT));
  s.w_lane = w0 + gl * 4 * static_cast<int>(sizeof(WT));
  s.g_lane = g0 + gl * 4 * static_cast<int>(sizeof(GT));
  s.mbase = p.optimizer == B200TBE_OPT_ROWWISE_ADAGRAD ? p.momentum1 + __ldg(p.momentum1_offsets + t) : nullptr;
  s.bag0 = static_cast<uint32_t>(t) * static_cast<uint32_t>(p.B);
  s.gstride_bytes = p.grad_stride * static_cast<int64_t>(sizeof(GT));
  s.row_bytes = s.D * static_cast<int>(sizeof(WT));
  // a quad is 16 bytes of a float row, 8 of a half row; slice offsets travel in 16-byte units
  s.ok = s.D > 0 && (s.D & 3) == 0 && s.D <= GS * kC * 4 &&
         (reinterpret_cast<uintptr_t>(w0) & (4 * sizeof(WT) - 1)) == 0 &&
         (reinterpret_cast<uintptr_t>(g0) & (4 * sizeof(GT) - 1)) == 0 && (s.gstride_bytes & 15) == 0;
  return s;
}

// The optimizer step for the row whose summed gradient is in acc (complete in every lane of the
// group) and whose weights were loaded into wv. sq = sum of squares of the gradient. Only lanes
// with write set store.
template <typename WT, int kC>
__device__ __forceinline__ void sweep_update(const BwdDev& p, const float4 (&acc)[kC],
                                             const typename Quad<WT>::Raw (&wv)[kC], const bool (&on)[kC],
                                             float sq, float m_old, float* mptr, char* wrow, float inv_D,
                                             int quad_w, bool write, bool first_lane) {
  float step = p.learning_rate;
  if (p.optimizer == B200TBE_OPT_ROWWISE_ADAGRAD) {
    const float m_new = fmaf(sq, inv_D, m_old);   // m += mean of the squares
    if (write && first_lane) *mptr = m_new;
    step = __fdividef(p.learning_rate, sqrt_fast(m_new) + p.eps);
  }
#pragma unroll
  for (int c = 0; c < kC; ++c) {
    if (write && on[c]) {
      float4 w = Quad<WT>::to(wv[c]);
      w.x = fmaf(-step, acc[c].x, w.x);
      w.y = fmaf(-step, acc[c].y, w.y);
      w.z = fmaf(-step, acc[c].z, w.z);
      w.w = fmaf(-step, acc[c].w, w.w);
      Quad<WT>::store(wrow + c * quad_w, w);
    }
  }
}

template <int kC>
__device__ __forceinline__ float sum_squares(const float4 (&acc)[kC]) {
  float sq = 0.f;
#pragma unroll
  for (int c = 0; c < kC; ++c) {
    sq = fmaf(acc[c].x, acc[c].x, sq);
    sq = fmaf(acc[c].y, acc[c].y, sq);
    sq = fmaf(acc[c].z, acc[c].z, sq);
    sq = fmaf(acc[c].w, acc[c].w, sq);
  }
  return sq;
}

template <int kC>
__device__ __forceinline__ void store_partial(float* dst, const float4 (&acc)[kC], const bool (&on)[kC],
                                              int gl, int GS) {
#pragma unroll
  for (int c = 0; c < kC; ++c)
    if (on[c]) *reinterpret_cast<float4*>(dst + (c * GS + gl) * 4) = acc[c];
}

struct SweepMeta {
  uint32_t row;    // row id of the position
  uint32_t goff;   // offset of its gradient slice in 16-byte units, kNoSlice for a skipped lookup
  float mult;      // factor of the slice (per-sample weight, 1 / bag length)
  bool tail;       // the position ends a run of several lookups
  bool single;     // the position is a whole run: the row's only lookup
};

// Where a group's span lies (per lane; spans of one warp are consecutive and share the table).
struct SpanCtx {
  uint32_t span_id;
  uint32_t s_begin;     // first sorted position of the span
  int s_count;          // positions in the span (0: this group has none)
  int cnt0;             // positions in the warp's first span (the longest of the warp)
  uint32_t seg_begin, seg_end;   // the table's sorted positions
  int grp, gl;
};

// kFull: the table's rows fill the group exactly (D = GS * kC * 4), so no lane ever sits out.
template <typename WT, typename GT, bool kScaled, int GS, int kC, bool kFull, int kSweepLoads>
__device__ __forceinline__ void sweep_span(const BwdDev& p, const SpanCtx& sc, const SweepTable<WT, GT>& tab) {
  constexpr int NG = 32 / GS;
  constexpr uint32_t kGroupBits = GS == 32 ? 1u : (GS == 16 ? 0x00010001u : 0x01010101u);
  constexpr uint32_t kBlockBits = kGroupBits * ((1u << kSweepLoads) - 1u);
  constexpr int quad_w = GS * 4 * static_cast<int>(sizeof(WT));   // bytes between a lane's quads
  constexpr int quad_g = GS * 4 * static_cast<int>(sizeof(GT));
  const int grp = sc.grp, gl = sc.gl;
  const uint32_t s_begin = sc.s_begin, seg_begin = sc.seg_begin, seg_end = sc.seg_end;
  const int s_count = sc.s_count, cnt0 = sc.cnt0;
  const uint32_t* __restrict__ keys = reinterpret_cast<const uint32_t*>(p.sorted_keys);
  const uint32_t* __restrict__ vals = p.sorted_vals;

  bool on[kC];
#pragma unroll
  for (int c = 0; c < kC; ++c) on[c] = kFull || (c * GS + gl) * 4 < tab.D;

  // does the span begin inside a run, does it end inside one?
  bool first_pending = false, tail_open = false;
  if (s_count > 0) {
    if (s_begin > seg_begin) first_pending = __ldg(keys + s_begin - 1) == __ldg(keys + s_begin);
    const uint32_t last = s_begin + s_count - 1;
    if (last + 1 < seg_end) tail_open = __ldg(keys + last) == __ldg(keys + last + 1);
  }

  const uint32_t gstride16 = static_cast<uint32_t>(tab.gstride_bytes >> 4);
  const char* w_row0 = tab.w_lane - gl * 4 * static_cast<int>(sizeof(WT));
  const float inv_D = 1.f / static_cast<float>(tab.D);

  // Three batches are in the pipe: the ids and bag ids of batch b + 2 are being loaded, batch
  // b + 1 is being turned into slice offsets (and the rows of the runs that end in it are asked
  // from L2), batch b is being summed. No step waits on a load issued in the same step.
  struct Raw {
    uint32_t key, next, prev, payload;
  };
  auto load_raw = [&](int b) {
    Raw r;
    const int i = b + gl;
    const uint32_t pos = s_begin + i;
    r.key = 0;
    r.next = 0xffffffffu;
    r.prev = 0xffffffffu;
    r.payload = kInvalidPayload;
    if (i < s_count) {
      r.key = __ldg(keys + pos);
      if (pos + 1 < seg_end) r.next = __ldg(keys + pos + 1);
      if (pos > seg_begin) r.prev = __ldg(keys + pos - 1);
      r.payload = __ldg(vals + pos);
    }
    return r;
  };
  auto derive = [&](const Raw& r, int b) {
    SweepMeta m;
    const int i = b + gl;
    const bool valid = i < s_count;
    const uint32_t pos = s_begin + i;
    m.row = r.key;
    m.goff = kNoSlice;
    m.mult = 1.f;
    // the table's first / last position begins / ends a run whatever lies beside it in memory
    const bool ends = valid && (pos + 1 >= seg_end || r.next != r.key);
    const bool begins = valid && (pos <= seg_begin || r.prev != r.key);
    if (valid && r.payload != kInvalidPayload) {
      int64_t bag = r.payload;
      if (kScaled) {
        if (p.per_sample_weights != nullptr) {
          m.mult = __ldg(p.per_sample_weights + r.payload);
          bag = __ldg(p.bag_of_pos + r.payload);
        }
        if (p.pooling_mode == B200TBE_POOL_MEAN) m.mult /= static_cast<float>(bag_length(p, bag));
      }
      m.goff = static_cast<uint32_t>((bag - tab.bag0) * gstride16);
    }
    // a run of one lookup needs no summing: it is updated in the singles pass of its batch (a
    // skipped lookup that is alone on its row needs nothing at all)
    m.single = NG > 1 && begins && ends && m.goff != kNoSlice;
    m.tail = ends && !m.single && (NG == 1 || !begins);
    if (m.single || m.tail) {
      // the row's weights and state start their way from HBM now, a batch ahead of the update
      const char* w = w_row0 + static_cast<uint64_t>(m.row) * static_cast<uint32_t>(tab.row_bytes);
      for (int off = 0; off < tab.row_bytes; off += 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(w + off));
      if (tab.mbase != nullptr) asm volatile("prefetch.global.L2 [%0];" ::"l"(tab.mbase + m.row));
    }
    return m;
  };
  float4 acc[kC];
#pragma unroll
  for (int c = 0; c < kC; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);

  SweepMeta cur = derive(load_raw(0), 0);
  Raw raw1 = load_raw(GS);
  for (int b = 0; b < cnt0; b += GS) {
    const Raw raw2 = load_raw(b + 2 * GS);
    const SweepMeta nxt = derive(raw1, b + GS);
    const uint32_t tailmask = __ballot_sync(kFullMask, cur.tail);
    // positions the sweep has to visit: lookups of runs of several lookups
    const uint32_t goff_sweep = cur.single ? kNoSlice : cur.goff;
    const uint32_t sliced = __ballot_sync(kFullMask, goff_sweep != kNoSlice);
    const uint32_t work = sliced | tailmask;
    const int nsteps = cnt0 - b < GS ? cnt0 - b : GS;
    for (int j0 = 0; j0 < nsteps; j0 += kSweepLoads) {
      if (((work >> j0) & kBlockBits) == 0) continue;   // nothing but one-lookup runs here
      // gradient slices of the next kSweepLoads positions: all requested before the first is added.
      // The usual block -- every position of every group has a slice -- loads without a test.
      typename Quad<GT>::Raw x[kSweepLoads][kC];
      float mu[kSweepLoads];
      const bool all_sliced = kFull && ((~sliced >> j0) & kBlockBits) == 0;
      if (all_sliced) {
#pragma unroll
        for (int u = 0; u < kSweepLoads; ++u) {
          const uint32_t off = __shfl_sync(kFullMask, goff_sweep, j0 + u, GS);   // j0 + u < GS
          mu[u] = 1.f;
          if (kScaled) mu[u] = __shfl_sync(kFullMask, cur.mult, j0 + u, GS);
          const char* src = tab.g_lane + (static_cast<uint64_t>(off) << 4);
#pragma unroll
          for (int c = 0; c < kC; ++c) x[u][c] = Quad<GT>::load_ro(src + c * quad_g);
        }
      } else {
#pragma unroll
        for (int u = 0; u < kSweepLoads; ++u) {
          const uint32_t off = __shfl_sync(kFullMask, goff_sweep, j0 + u, GS);
          mu[u] = 1.f;
          if (kScaled) mu[u] = __shfl_sync(kFullMask, cur.mult, j0 + u, GS);
          const char* src = tab.g_lane + (static_cast<uint64_t>(off) << 4);
#pragma unroll
          for (int c = 0; c < kC; ++c) {
            x[u][c] = Quad<GT>::zero();
            if (off != kNoSlice && on[c]) x[u][c] = Quad<GT>::load_ro(src + c * quad_g);
          }
        }
      }
      if (((tailmask >> j0) & kBlockBits) == 0) {
        // no run of any group ends among these positions (always so inside a long run): just add
#pragma unroll
        for (int u = 0; u < kSweepLoads; ++u) {
#pragma unroll
          for (int c = 0; c < kC; ++c) {
            if (kScaled) {
              const float4 f = Quad<GT>::to(x[u][c]);
              acc[c].x = fmaf(f.x, mu[u], acc[c].x);
              acc[c].y = fmaf(f.y, mu[u], acc[c].y);
              acc[c].z = fmaf(f.z, mu[u], acc[c].z);
              acc[c].w = fmaf(f.w, mu[u], acc[c].w);
            } else {
              Quad<GT>::add(acc[c], x[u][c]);
            }
          }
        }
        continue;
      }
      // every run of this group that ends among these positions: its row's weights and state are
      // requested now, so that the updates below wait for one round trip together, not one each
      typename Quad<WT>::Raw wv[kSweepLoads][kC];
      float m_old[kSweepLoads];
      uint32_t rows[kSweepLoads];
#pragma unroll
      for (int u = 0; u < kSweepLoads; ++u) {
        rows[u] = 0;
        m_old[u] = 0.f;
#pragma unroll
        for (int c = 0; c < kC; ++c) wv[u][c] = Quad<WT>::zero();
        if (((tailmask >> (j0 + u)) & kGroupBits) == 0) continue;
        rows[u] = __shfl_sync(kFullMask, cur.row, j0 + u, GS);
        if ((tailmask >> (grp * GS + j0 + u)) & 1u) {
          const char* wrow = tab.w_lane + static_cast<uint64_t>(rows[u]) * static_cast<uint32_t>(tab.row_bytes);
#pragma unroll
          for (int c = 0; c < kC; ++c)
            if (on[c]) wv[u][c] = Quad<WT>::load(wrow + c * quad_w);
          if (tab.mbase != nullptr) m_old[u] = tab.mbase[rows[u]];
        }
      }
#pragma unroll
      for (int u = 0; u < kSweepLoads; ++u) {
        const int j = j0 + u;
#pragma unroll
        for (int c = 0; c < kC; ++c) {
          if (kScaled) {
            const float4 f = Quad<GT>::to(x[u][c]);
            acc[c].x = fmaf(f.x, mu[u], acc[c].x);
            acc[c].y = fmaf(f.y, mu[u], acc[c].y);
            acc[c].z = fmaf(f.z, mu[u], acc[c].z);
            acc[c].w = fmaf(f.w, mu[u], acc[c].w);
          } else {
            Quad<GT>::add(acc[c], x[u][c]);
          }
        }
        if (((tailmask >> j) & kGroupBits) == 0) continue;   // no group's run ends here
        // ---- a run ends at position j of some group ----
        const bool mine = (tailmask >> (grp * GS + j)) & 1u;
        float sq = sum_squares<kC>(acc);
#pragma unroll
        for (int o = GS >> 1; o > 0; o >>= 1) sq += __shfl_xor_sync(kFullMask, sq, o);
        if (mine) {
          if (first_pending) {
            store_partial<kC>(p.partials + static_cast<int64_t>(2 * sc.span_id) * p.max_D, acc, on, gl, GS);
            first_pending = false;
          } else if (sq != 0.f) {
            // an all-zero sum (only skipped lookups, or gradients that are zero) leaves the row as it is
            char* wrow = tab.w_lane + static_cast<uint64_t>(rows[u]) * static_cast<uint32_t>(tab.row_bytes);
            sweep_update<WT, kC>(p, acc, wv[u], on, sq, m_old[u], tab.mbase + rows[u], wrow, inv_D, quad_w, true,
                                 gl == 0);
          }
#pragma unroll
          for (int c = 0; c < kC; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
    }

    // ---- the batch's runs of one lookup: NG of them per step, one per group, whichever group's span
    // they lie in (a tile's spans share the table), two steps' loads in flight ----
    uint32_t singles = __ballot_sync(kFullMask, cur.single);
    while (singles != 0) {
      constexpr int kRounds = 2;
      int from[kRounds];
#pragma unroll
      for (int r = 0; r < kRounds; ++r) {
        from[r] = -1;
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          const int l = __ffs(singles) - 1;   // -1 once the mask is empty
          singles &= singles - 1;
          if (g == grp) from[r] = l;
        }
      }
      typename Quad<GT>::Raw x[kRounds][kC];
      typename Quad<WT>::Raw wv[kRounds][kC];
      float mu[kRounds], m_old[kRounds];
      uint32_t rows[kRounds];
#pragma unroll
      for (int r = 0; r < kRounds; ++r) {
        const uint32_t off = __shfl_sync(kFullMask, cur.goff, from[r] & 31);
        rows[r] = __shfl_sync(kFullMask, cur.row, from[r] & 31);
        mu[r] = 1.f;
        if (kScaled) mu[r] = __shfl_sync(kFullMask, cur.mult, from[r] & 31);
        m_old[r] = 0.f;
        const char* src = tab.g_lane + (static_cast<uint64_t>(off) << 4);
        const char* wrow = tab.w_lane + static_cast<uint64_t>(rows[r]) * static_cast<uint32_t>(tab.row_bytes);
#pragma unroll
        for (int c = 0; c < kC; ++c) {
          x[r][c] = Quad<GT>::zero();
          wv[r][c] = Quad<WT>::zero();
          if (from[r] >= 0 && on[c]) {
            x[r][c] = Quad<GT>::load_ro(src + c * quad_g);
            wv[r][c] = Quad<WT>::load(wrow + c * quad_w);
          }
        }
        if (from[r] >= 0 && tab.mbase != nullptr) m_old[r] = tab.mbase[rows[r]];
      }
#pragma unroll
      for (int r = 0; r < kRounds; ++r) {
        float4 g1[kC];
#pragma unroll
        for (int c = 0; c < kC; ++c) {
          g1[c] = Quad<GT>::to(x[r][c]);
          if (kScaled) {
            g1[c].x *= mu[r];
            g1[c].y *= mu[r];
            g1[c].z *= mu[r];
            g1[c].w *= mu[r];
          }
        }
        float sq = sum_squares<kC>(g1);
#pragma unroll
        for (int o = GS >> 1; o > 0; o >>= 1) sq += __shfl_xor_sync(kFullMask, sq, o);
        if (from[r] >= 0 && sq != 0.f) {
          char* wrow = tab.w_lane + static_cast<uint64_t>(rows[r]) * static_cast<uint32_t>(tab.row_bytes);
          sweep_update<WT, kC>(p, g1, wv[r], on, sq, m_old[r], tab.mbase + rows[r], wrow, inv_D, quad_w, true,
                               gl == 0);
        }
      }
    }
    cur = nxt;
    raw1 = raw2;
  }

  if (s_count > 0) {
    uint32_t flags = 0;
    if (tail_open) {
      flags = first_pending ? kSpanThrough : kSpanTailOwner;
      float* dst = p.partials + static_cast<int64_t>(2 * sc.span_id + (first_pending ? 0 : 1)) * p.max_D;
      store_partial<kC>(dst, acc, on, gl, GS);
    }
    if (gl == 0) p.span_flags[sc.span_id] = flags;
  }
}

template <typename WT, typename GT, bool kScaled, int GS, int kC, int kMinCtas, int kLoads = sweep_loads_for<WT, GT, kScaled, kC, GS>()>
__global__ void __launch_bounds__(kSweepThreads, kMinCtas)
    sweep_runs_kernel(const __grid_constant__ BwdDev p) {
  constexpr int NG = 32 / GS;
  constexpr int kSpansPerCta = kSweepWarps * NG;
  static_assert(kSpansPerTile % kSpansPerCta == 0, "a CTA's spans lie in one tile");
  constexpr int kCtasPerTile = kSpansPerTile / kSpansPerCta;

  const uint32_t tile = blockIdx.x / kCtasPerTile;
  if (tile >= __ldg(p.total_tiles)) return;
  const uint4 td = __ldg(p.tile_desc + tile);   // {begin, count, table, first tile of the table}
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  SpanCtx sc;
  sc.grp = lane / GS;
  sc.gl = lane % GS;
  const int warp_span0 = static_cast<int>(blockIdx.x % kCtasPerTile) * kSpansPerCta + warp * NG;
  const int tile_n = static_cast<int>(td.y);
  if (warp_span0 * kSpan >= tile_n) return;
  const int span_in_tile = warp_span0 + sc.grp;
  sc.span_id = tile * kSpansPerTile + span_in_tile;
  const int t = static_cast<int>(td.z);
  const int s_off = span_in_tile * kSpan;
  sc.s_count = s_off >= tile_n ? 0 : (tile_n - s_off < kSpan ? tile_n - s_off : kSpan);
  sc.cnt0 = tile_n - warp_span0 * kSpan < kSpan ? tile_n - warp_span0 * kSpan : kSpan;
  sc.s_begin = td.x + s_off;
  sc.seg_begin = __ldg(p.seg_start + t);
  sc.seg_end = __ldg(p.seg_start + t + 1);

  const SweepTable<WT, GT> tab = sweep_table<WT, GT, GS, kC>(p, t, sc.gl);
  if (!tab.ok) {
    if (lane == 0 && p.status != nullptr) atomicOr(p.status, B200TBE_DEV_UNSUPPORTED_SHAPE);
    if (sc.gl == 0 && sc.s_count > 0) p.span_flags[sc.span_id] = 0;
    return;
  }
  if (tab.D == GS * kC * 4) {
    sweep_span<WT, GT, kScaled, GS, kC, true, kLoads>(p, sc, tab);
  } else {
    sweep_span<WT, GT, kScaled, GS, kC, false, kLoads>(p, sc, tab);
  }
}

// One warp per span whose last run continues to the right: adds the run's pieces in span order --
// the span's tail slot, then the head slot of every following span up to and including the first
// one that the run does not pass through -- and updates the row. Group g takes pieces g, g + NG, ...
template <typename WT, int GS, int kC>
__global__ void __launch_bounds__(kFinishWarps * 32)
    finish_open_runs_kernel(const __grid_constant__ BwdDev p) {
  constexpr int NG = 32 / GS;
  constexpr int quad_w = GS * 4 * static_cast<int>(sizeof(WT));
  const int lane = threadIdx.x & 31;
  const int grp = lane / GS, gl = lane % GS;
  const uint32_t span = blockIdx.x * kFinishWarps + (threadIdx.x >> 5);
  const uint32_t tile = span / kSpansPerTile;
  const uint32_t live_tiles = __ldg(p.total_tiles);
  if (tile >= live_tiles) return;
  const uint4 td = __ldg(p.tile_desc + tile);
  const int s_off = static_cast<int>(span % kSpansPerTile) * kSpan;
  if (s_off >= static_cast<int>(td.y)) return;
  if ((p.span_flags[span] & kSpanTailOwner) == 0) return;
  const int s_count = static_cast<int>(td.y) - s_off < kSpan ? static_cast<int>(td.y) - s_off : kSpan;
  const int t = static_cast<int>(td.z);

  // pieces after the tail slot: one per following span, the last being the first span that is not
  // passed through (flags of spans the run cannot reach are never decisive)
  const uint32_t span_limit = live_tiles * kSpansPerTile;
  uint32_t heads = 0;
  for (uint32_t v = span + 1;; v += 32) {
    const uint32_t mine = v + lane;
    const bool through = mine < span_limit && (p.span_flags[mine] & kSpanThrough) != 0;
    const uint32_t stop = __ballot_sync(kFullMask, !through);
    if (stop != 0) {
      heads += __ffs(stop);
      break;
    }
    heads += 32;
  }

  const int D_begin = __ldg(p.D_offsets + t);
  const int D = __ldg(p.D_offsets + t + 1) - D_begin;
  bool on[kC];
  float4 acc[kC];
#pragma unroll
  for (int c = 0; c < kC; ++c) {
    on[c] = (c * GS + gl) * 4 < D;
    acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // piece 0 = tail slot of `span`; piece i >= 1 = head slot of span + i. A row looked up 150 000
  // times leaves almost 600 pieces to one warp, so eight pieces are requested before the first is
  // added (the additions keep their order).
  constexpr int kPieces = 8 / kC;
  const float* lane_base = p.partials + (gl * 4);
  auto slot_of = [&](uint32_t i) -> int64_t {
    return i == 0 ? 2 * static_cast<int64_t>(span) + 1 : 2 * static_cast<int64_t>(span + i);
  };
  for (uint32_t i0 = grp; i0 <= heads; i0 += NG * kPieces) {
    float4 x[kPieces][kC];
#pragma unroll
    for (int u = 0; u < kPieces; ++u) {
      const uint32_t i = i0 + u * NG;
      const float* src = lane_base + slot_of(i <= heads ? i : i0) * p.max_D;
#pragma unroll
      for (int c = 0; c < kC; ++c) {
        x[u][c] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i <= heads && on[c]) x[u][c] = *reinterpret_cast<const float4*>(src + c * GS * 4);
      }
    }
#pragma unroll
    for (int u = 0; u < kPieces; ++u) {
#pragma unroll
      for (int c = 0; c < kC; ++c) {
        acc[c].x += x[u][c].x;
        acc[c].y += x[u][c].y;
        acc[c].z += x[u][c].z;
        acc[c].w += x[u][c].w;
      }
    }
  }
#pragma unroll
  for (int o = GS; o < 32; o <<= 1) {
#pragma unroll
    for (int c = 0; c < kC; ++c) {
      acc[c].x += __shfl_xor_sync(kFullMask, acc[c].x, o);
      acc[c].y += __shfl_xor_sync(kFullMask, acc[c].y, o);
      acc[c].z += __shfl_xor_sync(kFullMask, acc[c].z, o);
      acc[c].w += __shfl_xor_sync(kFullMask, acc[c].w, o);
    }
  }
  float sq = sum_squares<kC>(acc);
#pragma unroll
  for (int o = GS >> 1; o > 0; o >>= 1) sq += __shfl_xor_sync(kFullMask, sq, o);
  if (sq == 0.f) return;
  const uint32_t row = __ldg(reinterpret_cast<const uint32_t*>(p.sorted_keys) + td.x + s_off + s_count - 1);
  char* wrow = p.dev_weights + (__ldg(p.weights_offsets + t) + static_cast<int64_t>(row) * D) * static_cast<int64_t>(sizeof(WT)) +
               gl * 4 * static_cast<int>(sizeof(WT));
  float* mptr = nullptr;
  float m_old = 0.f;
  if (p.optimizer == B200TBE_OPT_ROWWISE_ADAGRAD) {
    mptr = p.momentum1 + __ldg(p.momentum1_offsets + t) + row;
    m_old = *mptr;
  }
  typename Quad<WT>::Raw wv[kC];
#pragma unroll
  for (int c = 0; c < kC; ++c) {
    wv[c] = Quad<WT>::zero();
    if (grp == 0 && on[c]) wv[c] = Quad<WT>::load(wrow + c * quad_w);
  }
  sweep_update<WT, kC>(p, acc, wv, on, sq, m_old, mptr, wrow, 1.f / static_cast<float>(D), quad_w, grp == 0, gl == 0);
}
