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
//   * a run that crosses a span boundary leaves partial sums in scratch instead (the piece that
//     ends a run begun earlier -> "head" slot of the span, the piece that begins a run finished
//     later -> "tail" slot); finish_open_runs_kernel adds a run's pieces in span order and updates.
// Nothing depends on scheduling: the order of additions is fixed by the sorted order alone.
//
// Part of tbe_backward.cu: included there inside its namespace, after BwdDev and bag_length.
#pragma once

constexpr int kSpan = 256;                                  // sorted positions per span
constexpr int kSpansPerTile = kSortPlanTile / kSpan;        // 16
constexpr int kSweepWarps = 4;
constexpr int kSweepThreads = kSweepWarps * 32;
// positions whose gradient slices are in flight per group (fewer when a lane holds more of a row)
template <int kC>
__host__ __device__ constexpr int sweep_loads() {
  return kC <= 2 ? 4 : 2;
}
template <typename GT, int kC>
__host__ __device__ constexpr int sweep_ctas_per_sm() {
  return kC > 2 ? 5 : 8;
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
  for (uint32_t base = 0; base < total; base += 32) {
    const uint32_t rel = base + lane;
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
      int64_t idx = load_index<IndexT>(p.indices, j);
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
                                             float sq, float m_old, float* mptr, char* wrow, int D,
                                             int quad_w, bool write, bool first_lane) {
  float step = p.learning_rate;
  if (p.optimizer == B200TBE_OPT_ROWWISE_ADAGRAD) {
    const float m_new = m_old + sq / static_cast<float>(D);
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
  bool tail;       // the position ends a run
};

template <typename WT, typename GT, bool kScaled, int GS, int kC, int kMinCtas>
__global__ void __launch_bounds__(kSweepThreads, kMinCtas)
    sweep_runs_kernel(const __grid_constant__ BwdDev p) {
  constexpr int NG = 32 / GS;
  constexpr int kSweepLoads = sweep_loads<kC>();
  constexpr int kSpansPerCta = kSweepWarps * NG;
  static_assert(kSpansPerTile % kSpansPerCta == 0, "a CTA's spans lie in one tile");
  constexpr int kCtasPerTile = kSpansPerTile / kSpansPerCta;
  constexpr uint32_t kGroupBits = GS == 32 ? 1u : (GS == 16 ? 0x00010001u : 0x01010101u);
  constexpr int quad_w = GS * 4 * static_cast<int>(sizeof(WT));   // bytes between a lane's quads
  constexpr int quad_g = GS * 4 * static_cast<int>(sizeof(GT));

  const uint32_t tile = blockIdx.x / kCtasPerTile;
  if (tile >= __ldg(p.total_tiles)) return;
  const uint4 td = __ldg(p.tile_desc + tile);   // {begin, count, table, first tile of the table}
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grp = lane / GS, gl = lane % GS;
  const int warp_span0 = static_cast<int>(blockIdx.x % kCtasPerTile) * kSpansPerCta + warp * NG;
  const int tile_n = static_cast<int>(td.y);
  if (warp_span0 * kSpan >= tile_n) return;
  const int span_in_tile = warp_span0 + grp;
  const uint32_t span_id = tile * kSpansPerTile + span_in_tile;
  const int t = static_cast<int>(td.z);
  const int s_off = span_in_tile * kSpan;
  const int s_count = s_off >= tile_n ? 0 : (tile_n - s_off < kSpan ? tile_n - s_off : kSpan);
  const int cnt0 = tile_n - warp_span0 * kSpan < kSpan ? tile_n - warp_span0 * kSpan : kSpan;  // group 0: the longest
  const uint32_t s_begin = td.x + s_off;
  const uint32_t seg_begin = __ldg(p.seg_start + t), seg_end = __ldg(p.seg_start + t + 1);
  const uint32_t* __restrict__ keys = reinterpret_cast<const uint32_t*>(p.sorted_keys);
  const uint32_t* __restrict__ vals = p.sorted_vals;

  const SweepTable<WT, GT> tab = sweep_table<WT, GT, GS, kC>(p, t, gl);
  if (!tab.ok) {
    if (lane == 0 && p.status != nullptr) atomicOr(p.status, B200TBE_DEV_UNSUPPORTED_SHAPE);
    if (gl == 0 && s_count > 0) p.span_flags[span_id] = 0;
    return;
  }
  bool on[kC];
#pragma unroll
  for (int c = 0; c < kC; ++c) on[c] = (c * GS + gl) * 4 < tab.D;

  // does the span begin inside a run, does it end inside one?
  bool first_pending = false, tail_open = false;
  if (s_count > 0) {
    if (s_begin > seg_begin) first_pending = __ldg(keys + s_begin - 1) == __ldg(keys + s_begin);
    const uint32_t last = s_begin + s_count - 1;
    if (last + 1 < seg_end) tail_open = __ldg(keys + last) == __ldg(keys + last + 1);
  }

  auto load_meta = [&](int b) {
    SweepMeta m;
    const int i = b + gl;
    const bool valid = i < s_count;
    const uint32_t pos = s_begin + i;
    m.row = 0;
    m.goff = kNoSlice;
    m.mult = 1.f;
    m.tail = false;
    if (valid) {
      m.row = __ldg(keys + pos);
      const bool last_of_table = pos + 1 >= seg_end;
      const uint32_t next = last_of_table ? 0u : __ldg(keys + pos + 1);
      m.tail = last_of_table || next != m.row;
      const uint32_t payload = __ldg(vals + pos);
      if (payload != kInvalidPayload) {
        int64_t bag = payload;
        if (kScaled) {
          if (p.per_sample_weights != nullptr) {
            m.mult = __ldg(p.per_sample_weights + payload);
            bag = __ldg(p.bag_of_pos + payload);
          }
          if (p.pooling_mode == B200TBE_POOL_MEAN) m.mult /= static_cast<float>(bag_length(p, bag));
        }
        m.goff = static_cast<uint32_t>(((bag - tab.bag0) * tab.gstride_bytes) >> 4);
      }
      if (m.tail) {
        // the row's weights and state start their way from HBM now, a batch ahead of the update
        const char* w = tab.w_lane - gl * 4 * static_cast<int>(sizeof(WT)) +
                        static_cast<uint64_t>(m.row) * static_cast<uint32_t>(tab.row_bytes);
        if (p.tune_prefetch_l1) {
          for (int off = 0; off < tab.row_bytes; off += 128)
            asm volatile("prefetch.global.L1 [%0];" ::"l"(w + off));
          if (tab.mbase != nullptr) asm volatile("prefetch.global.L1 [%0];" ::"l"(tab.mbase + m.row));
        } else {
          for (int off = 0; off < tab.row_bytes; off += 128)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(w + off));
          if (tab.mbase != nullptr) asm volatile("prefetch.global.L2 [%0];" ::"l"(tab.mbase + m.row));
        }
      }
    }
    return m;
  };

  float4 acc[kC];
#pragma unroll
  for (int c = 0; c < kC; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);

  SweepMeta cur = load_meta(0);
  for (int b = 0; b < cnt0; b += GS) {
    const SweepMeta nxt = load_meta(b + GS);
    const uint32_t tailmask = __ballot_sync(kFullMask, cur.tail);
    const int nsteps = cnt0 - b < GS ? cnt0 - b : GS;
    for (int j0 = 0; j0 < nsteps; j0 += kSweepLoads) {
      typename Quad<GT>::Raw x[kSweepLoads][kC];
      float mu[kSweepLoads];
#pragma unroll
      for (int u = 0; u < kSweepLoads; ++u) {
        const int j = j0 + u;   // < GS: kSweepLoads divides GS
        const uint32_t off = __shfl_sync(kFullMask, cur.goff, j, GS);
        mu[u] = 1.f;
        if (kScaled) mu[u] = __shfl_sync(kFullMask, cur.mult, j, GS);
        const char* src = tab.g_lane + (static_cast<uint64_t>(off) << 4);
#pragma unroll
        for (int c = 0; c < kC; ++c) {
          x[u][c] = Quad<GT>::zero();
          if (off != kNoSlice && on[c]) x[u][c] = Quad<GT>::load_ro(src + c * quad_g);
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
        const uint32_t row = __shfl_sync(kFullMask, cur.row, j, GS);
        const bool upd = mine && !first_pending;
        char* wrow = tab.w_lane + static_cast<uint64_t>(row) * static_cast<uint32_t>(tab.row_bytes);
        typename Quad<WT>::Raw wv[kC];
        float m_old = 0.f;
#pragma unroll
        for (int c = 0; c < kC; ++c) {
          wv[c] = Quad<WT>::zero();
          if (upd && on[c]) wv[c] = Quad<WT>::load(wrow + c * quad_w);
        }
        if (upd && tab.mbase != nullptr) m_old = tab.mbase[row];
        float sq = sum_squares<kC>(acc);
#pragma unroll
        for (int o = GS >> 1; o > 0; o >>= 1) sq += __shfl_xor_sync(kFullMask, sq, o);
        if (mine) {
          if (first_pending) {
            store_partial<kC>(p.partials + static_cast<int64_t>(2 * span_id) * p.max_D, acc, on, gl, GS);
            first_pending = false;
          } else if (sq != 0.f) {
            // an all-zero sum (only skipped lookups, or gradients that are zero) leaves the row as it is
            sweep_update<WT, kC>(p, acc, wv, on, sq, m_old, tab.mbase + row, wrow, tab.D, quad_w, true, gl == 0);
          }
#pragma unroll
          for (int c = 0; c < kC; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
    }
    cur = nxt;
  }

  if (s_count > 0) {
    uint32_t flags = 0;
    if (tail_open) {
      flags = first_pending ? kSpanThrough : kSpanTailOwner;
      float* dst = p.partials + static_cast<int64_t>(2 * span_id + (first_pending ? 0 : 1)) * p.max_D;
      store_partial<kC>(dst, acc, on, gl, GS);
    }
    if (gl == 0) p.span_flags[span_id] = flags;
  }
}

// One warp per span whose last run continues to the right: adds the run's pieces in span order --
// the span's tail slot, then the head slot of every following span up to and including the first
// one that the run does not pass through -- and updates the row. Group g takes pieces g, g + NG, ...
template <typename WT, int GS, int kC>
__global__ void __launch_bounds__(kSweepThreads)
    finish_open_runs_kernel(const __grid_constant__ BwdDev p) {
  constexpr int NG = 32 / GS;
  constexpr int quad_w = GS * 4 * static_cast<int>(sizeof(WT));
  const int lane = threadIdx.x & 31;
  const int grp = lane / GS, gl = lane % GS;
  const uint32_t span = blockIdx.x * kSweepWarps + (threadIdx.x >> 5);
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
  // piece 0 = tail slot of `span`; piece i >= 1 = head slot of span + i
  const float* lane_base = p.partials + (gl * 4);
  for (uint32_t i = grp; i <= heads; i += NG) {
    const int64_t slot = i == 0 ? 2 * static_cast<int64_t>(span) + 1 : 2 * static_cast<int64_t>(span + i);
    const float* src = lane_base + slot * p.max_D;
#pragma unroll
    for (int c = 0; c < kC; ++c) {
      if (on[c]) {
        const float4 x = *reinterpret_cast<const float4*>(src + c * GS * 4);
        acc[c].x += x.x;
        acc[c].y += x.y;
        acc[c].z += x.z;
        acc[c].w += x.w;
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
  sweep_update<WT, kC>(p, acc, wv, on, sq, m_old, mptr, wrow, D, quad_w, grp == 0, gl == 0);
}
