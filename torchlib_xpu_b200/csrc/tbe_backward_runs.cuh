// Backward, the run pass for rows of at most 256 elements: reduce the gradient slices of every run
// of equal sorted keys and apply the optimizer step to that row, once.
//
// Shape of the work (recommender id streams): three runs in four have a single lookup and nine in
// ten at most four, so the pass is a random read-modify-write of one weight row per run plus one
// gathered gradient slice per lookup, and what bounds it is how many of those are in flight. Hence
// a plain grid at high occupancy instead of a persistent pipeline:
//   * a warp owns 32 consecutive runs. Lane j loads run j's metadata once, coalesced: start, length,
//     key -> (table, row), first payload, and the row's weight / state / gradient-column pointers;
//   * a run is processed by a group of gs lanes, each holding kQ quads of 4 elements (quad
//     v + gs*k in lane v, so every load instruction of a group reads contiguous bytes); gs = 8 for
//     D = 128, and a warp works on 32/gs runs at once, which is what amortises the per-run scalar
//     work (shuffles, the optimizer's sqrt and divisions). The metadata reaches the group by
//     shuffle, the weights and optimizer state are loaded before the gradients are summed, and the
//     first gradient slice depends on no other load: payload 0 came with the metadata;
//   * later lookups of a run: the group's lanes fetch gs payloads with one coalesced load and hand
//     the gradient offsets round by shuffle;
//   * runs of more than kShortRun lookups would hold their group (and with it the warp and the
//     CTA's slot) for hundreds of dependent steps, so after the short runs the warp takes its
//     medium runs one at a time with all lanes: 32 payloads per fetch, the groups take every
//     (32/gs)-th lookup, the partial sums are combined across groups by shuffle;
//   * runs longer than kLongRun are recorded for the chunked path and skipped here.
// Summation order inside a run is the sorted (= original position) order, fixed by the data alone.
//
// Part of tbe_backward.cu: included there inside its namespace, after BwdDev and bag_length.
#pragma once

constexpr int kRunWarps = 4;       // small CTAs: a slot is held until the CTA's slowest warp is done
constexpr int kRunThreads = kRunWarps * 32;
constexpr int kRunCtasPerSm = 6;   // 24 warps per SM, 85 registers per thread
// The runs and chunks kernels with fp16 gradients (half the registers per gradient quad) measured 4 % faster at 8
// CTAs (64 registers, some spills) than at 6; with fp32 gradients 4 % slower.
template <typename GT>
constexpr int run_ctas_per_sm() {
  return sizeof(GT) == 2 ? 8 : kRunCtasPerSm;
}
constexpr int kShortRun = 16;      // longer runs are summed by the whole warp, one at a time
constexpr uint32_t kNoSlice = 0xffffffffu;

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
  // round to nearest even
  static __device__ __forceinline__ void store(char* p, float4 f) {
    *reinterpret_cast<uint2*>(p) = make_uint2(float2_to_half2_bits(f.x, f.y), float2_to_half2_bits(f.z, f.w));
  }
};

__device__ __forceinline__ unsigned long long shfl_ptr(const void* p, int src) {
  return __shfl_sync(kFullMask, reinterpret_cast<unsigned long long>(p), src);
}

// Everything a group needs to know about the run it works on.
struct RunView {
  uint32_t len, start, pay0, bag0;
  int D;
  char* w_lane;         // weights of the row, at this lane's first quad
  float* mptr;          // row-wise optimizer state, or null
  const char* g_lane;   // the table's gradient columns in bag 0 of the table, at this lane's first quad
};

// Payload of lookup pos of the run -> offset of its gradient slice in 16-byte units (kNoSlice for an
// out-of-range lookup) and the factor the slice is scaled by.
template <bool kScaled>
__device__ __forceinline__ uint32_t slice_of(const BwdDev& p, const RunView& r, uint32_t pos,
                                             int64_t gstride_bytes, float& mult) {
  mult = 1.f;
  if (pos >= r.len) return kNoSlice;
  const uint32_t payload = pos == 0 ? r.pay0 : __ldg(p.sorted_vals + r.start + pos);
  if (payload == kInvalidPayload) return kNoSlice;
  int64_t bag = payload;
  if (kScaled) {
    if (p.per_sample_weights != nullptr) {
      mult = __ldg(p.per_sample_weights + payload);
      bag = __ldg(p.bag_of_pos + payload);
    }
    if (p.pooling_mode == B200TBE_POOL_MEAN) mult /= static_cast<float>(bag_length(p, bag));
  }
  return static_cast<uint32_t>(((bag - r.bag0) * gstride_bytes) >> 4);
}

template <typename GT, bool kScaled, int kQ>
__device__ __forceinline__ void add_slice(float4 (&acc)[kQ], const bool (&on)[kQ], const char* g_lane,
                                          uint32_t ch, float m, int quad_step) {
  const char* src = g_lane + (static_cast<uint64_t>(ch) << 4);
  typename Quad<GT>::Raw x[kQ];
#pragma unroll
  for (int k = 0; k < kQ; ++k) {
    x[k] = Quad<GT>::zero();
    if (ch != kNoSlice && on[k]) x[k] = Quad<GT>::load_ro(src + k * quad_step);
  }
#pragma unroll
  for (int k = 0; k < kQ; ++k) {
    const float4 f = Quad<GT>::to(x[k]);
    if (kScaled) {
      acc[k].x = fmaf(f.x, m, acc[k].x);
      acc[k].y = fmaf(f.y, m, acc[k].y);
      acc[k].z = fmaf(f.z, m, acc[k].z);
      acc[k].w = fmaf(f.w, m, acc[k].w);
    } else {
      acc[k].x += f.x;
      acc[k].y += f.y;
      acc[k].z += f.z;
      acc[k].w += f.w;
    }
  }
}

// Whole warp on one run: group h sums lookups h, h + G, ... of the run and the groups' sums are
// added by shuffle, so every lane ends with the run's complete sum of its quads.
template <typename GT, bool kScaled, int kQ>
__device__ __forceinline__ void sum_whole_warp(const BwdDev& p, const RunView& run, float4 (&acc)[kQ],
                                               const bool (&on)[kQ], int64_t gstride_bytes, int lane,
                                               int h, int G, int gs, int quad_g) {
  for (uint32_t base = 0; base < run.len; base += 32) {
    float mult;
    const uint32_t goff = slice_of<kScaled>(p, run, base + lane, gstride_bytes, mult);
    const int n = run.len - base < 32u ? static_cast<int>(run.len - base) : 32;
    for (int j = h; j - h < n; j += G) {   // j - h is the same in every lane: the shuffles stay converged
      const uint32_t ch = __shfl_sync(kFullMask, goff, j & 31);
      float m = 1.f;
      if (kScaled) m = __shfl_sync(kFullMask, mult, j & 31);
      add_slice<GT, kScaled, kQ>(acc, on, run.g_lane, j < n ? ch : kNoSlice, m, quad_g);
    }
  }
  for (int o = gs; o < 32; o <<= 1) {
#pragma unroll
    for (int k = 0; k < kQ; ++k) {
      acc[k].x += __shfl_xor_sync(kFullMask, acc[k].x, o);
      acc[k].y += __shfl_xor_sync(kFullMask, acc[k].y, o);
      acc[k].z += __shfl_xor_sync(kFullMask, acc[k].z, o);
      acc[k].w += __shfl_xor_sync(kFullMask, acc[k].w, o);
    }
  }
}

// The optimizer step for the run summed in acc (complete in every lane of the group). Every lane
// runs this; only lanes with write set store.
template <typename WT, int kQ>
__device__ __forceinline__ void update_row(const BwdDev& p, const RunView& r, const float4 (&acc)[kQ],
                                           const typename Quad<WT>::Raw (&wv)[kQ], const bool (&on)[kQ],
                                           float m_old, bool write, int v, int gs, int quad_step) {
  float step = p.learning_rate;
  if (p.optimizer == B200TBE_OPT_ROWWISE_ADAGRAD) {
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < kQ; ++k) {
      sq = fmaf(acc[k].x, acc[k].x, sq);
      sq = fmaf(acc[k].y, acc[k].y, sq);
      sq = fmaf(acc[k].z, acc[k].z, sq);
      sq = fmaf(acc[k].w, acc[k].w, sq);
    }
    for (int o = gs >> 1; o > 0; o >>= 1) sq += __shfl_xor_sync(kFullMask, sq, o);
    const float m_new = m_old + sq / static_cast<float>(r.D);
    if (write && v == 0) *r.mptr = m_new;
    step = p.learning_rate / (sqrtf(m_new) + p.eps);
  }
#pragma unroll
  for (int k = 0; k < kQ; ++k) {
    if (write && on[k]) {
      float4 w = Quad<WT>::to(wv[k]);
      w.x = fmaf(-step, acc[k].x, w.x);
      w.y = fmaf(-step, acc[k].y, w.y);
      w.z = fmaf(-step, acc[k].z, w.z);
      w.w = fmaf(-step, acc[k].w, w.w);
      Quad<WT>::store(r.w_lane + k * quad_step, w);
    }
  }
}

template <typename KeyT, typename WT, typename GT, bool kScaled, int kQ>
__global__ void __launch_bounds__(kRunThreads, run_ctas_per_sm<GT>())
    reduce_runs_groups_kernel(const __grid_constant__ BwdDev p) {
  const int lane = threadIdx.x & 31;
  const int64_t runs = p.counters[0];
  const int64_t run0 = (static_cast<int64_t>(blockIdx.x) * kRunWarps + (threadIdx.x >> 5)) * 32;
  if (run0 >= runs) return;
  const int n_runs = runs - run0 < 32 ? static_cast<int>(runs - run0) : 32;
  const int gs = lanes_per_row((p.max_D + 4 * kQ - 1) / (4 * kQ));
  const int gshift = __ffs(gs) - 1;
  const int G = 32 >> gshift;   // runs in flight per warp
  const int h = lane >> gshift;
  const int v = lane & (gs - 1);
  const int64_t gstride_bytes = p.grad_stride * static_cast<int64_t>(sizeof(GT));
  const int quad_w = gs * 4 * static_cast<int>(sizeof(WT));   // bytes between a lane's quads, weights
  const int quad_g = gs * 4 * static_cast<int>(sizeof(GT));   // and gradients

  // ---- lane j describes run run0 + j ----
  RunView mine;
  mine.len = 0;
  mine.start = 0;
  mine.pay0 = kInvalidPayload;
  mine.bag0 = 0;
  mine.D = 0;
  mine.w_lane = nullptr;
  mine.mptr = nullptr;
  mine.g_lane = nullptr;
  bool my_medium = false;
  if (lane < n_runs) {
    mine.start = p.run_start[run0 + lane];
    mine.len = p.run_start[run0 + lane + 1] - mine.start;
    const int64_t key = static_cast<int64_t>(reinterpret_cast<const KeyT*>(p.sorted_keys)[mine.start]);
    mine.pay0 = p.sorted_vals[mine.start];
    int lo = 0, hi = p.T - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (__ldg(p.hash_size_cumsum + mid) <= key) {
        lo = mid;
      } else {
        hi = mid - 1;
      }
    }
    const int t = lo;
    const int64_t row = key - __ldg(p.hash_size_cumsum + t);
    const int D_begin = __ldg(p.D_offsets + t);
    const int D = __ldg(p.D_offsets + t + 1) - D_begin;
    mine.D = D;
    mine.w_lane = p.dev_weights + (__ldg(p.weights_offsets + t) + row * D) * static_cast<int64_t>(sizeof(WT));
    if (p.optimizer == B200TBE_OPT_ROWWISE_ADAGRAD)
      mine.mptr = p.momentum1 + __ldg(p.momentum1_offsets + t) + row;
    mine.g_lane = p.grad_output + (p.grad_col_offset + D_begin) * static_cast<int64_t>(sizeof(GT));
    mine.bag0 = static_cast<uint32_t>(t) * static_cast<uint32_t>(p.B);
    // a quad is 16 bytes of a float row, 8 of a half row; gradient offsets travel in 16-byte units
    const bool ok = D > 0 && (D & 3) == 0 && D <= gs * 4 * kQ &&
                    (reinterpret_cast<uintptr_t>(mine.w_lane) & (4 * sizeof(WT) - 1)) == 0 &&
                    (reinterpret_cast<uintptr_t>(mine.g_lane) & (4 * sizeof(GT) - 1)) == 0 &&
                    (gstride_bytes & 15) == 0;
    if (!ok) {
      if (p.status != nullptr) atomicOr(p.status, B200TBE_DEV_UNSUPPORTED_SHAPE);
      mine.len = 0;
    } else if (mine.len > static_cast<uint32_t>(kLongRun)) {
      const uint32_t chunks = (mine.len + kLongRun - 1) / kLongRun;
      const uint32_t slot = atomicAdd(p.counters + 1, 1u);
      const uint32_t chunk0 = atomicAdd(p.counters + 2, chunks);
      p.long_run[slot] = static_cast<uint32_t>(run0 + lane);
      p.long_chunk0[slot] = chunk0;
      for (uint32_t c = 0; c < chunks; ++c) p.chunk_run[chunk0 + c] = slot;
      mine.len = 0;
    } else {
      my_medium = mine.len > static_cast<uint32_t>(kShortRun);
      // all 32 rows of the warp start their way from HBM now; the groups reach them a few steps later
      for (int off = 0; off < D * static_cast<int>(sizeof(WT)); off += 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(mine.w_lane + off));
      if (mine.mptr != nullptr) asm volatile("prefetch.global.L2 [%0];" ::"l"(mine.mptr));
    }
  }
  uint32_t medium = __ballot_sync(kFullMask, my_medium);
  const uint32_t short_len = my_medium ? 0u : mine.len;

  auto view_of = [&](int r, uint32_t len) {
    RunView x;
    x.len = len;
    x.start = __shfl_sync(kFullMask, mine.start, r);
    x.pay0 = __shfl_sync(kFullMask, mine.pay0, r);
    x.bag0 = __shfl_sync(kFullMask, mine.bag0, r);
    x.D = __shfl_sync(kFullMask, mine.D, r);
    x.w_lane = reinterpret_cast<char*>(shfl_ptr(mine.w_lane, r)) + v * 4 * static_cast<int>(sizeof(WT));
    x.mptr = reinterpret_cast<float*>(shfl_ptr(mine.mptr, r));
    x.g_lane = reinterpret_cast<const char*>(shfl_ptr(mine.g_lane, r)) + v * 4 * static_cast<int>(sizeof(GT));
    return x;
  };

  // ---- short runs: one per group, G at a time ----
  for (int i = 0; i < n_runs; i += G) {
    const int r = i + h;   // < 32: G divides 32
    const uint32_t len = __shfl_sync(kFullMask, short_len, r);
    const uint32_t maxlen = __reduce_max_sync(kFullMask, len);
    if (maxlen == 0) continue;
    const RunView run = view_of(r, len);
    bool on[kQ];
    typename Quad<WT>::Raw wv[kQ];
#pragma unroll
    for (int k = 0; k < kQ; ++k) {
      on[k] = len > 0 && (v + gs * k) * 4 < run.D;
      wv[k] = Quad<WT>::zero();
      if (on[k]) wv[k] = Quad<WT>::load(run.w_lane + k * quad_w);
    }
    float m_old = 0.f;
    if (len > 0 && run.mptr != nullptr) m_old = *run.mptr;
    float4 acc[kQ];
#pragma unroll
    for (int k = 0; k < kQ; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t base = 0; base < maxlen; base += gs) {
      // lane v of the group fetches lookup base + v of the group's run
      float mult;
      const uint32_t goff = slice_of<kScaled>(p, run, base + v, gstride_bytes, mult);
      const int nmax = maxlen - base < static_cast<uint32_t>(gs) ? static_cast<int>(maxlen - base) : gs;
      for (int j = 0; j < nmax; ++j) {
        const uint32_t ch = __shfl_sync(kFullMask, goff, j, gs);
        float m = 1.f;
        if (kScaled) m = __shfl_sync(kFullMask, mult, j, gs);
        add_slice<GT, kScaled, kQ>(acc, on, run.g_lane, ch, m, quad_g);
      }
    }
    update_row<WT, kQ>(p, run, acc, wv, on, m_old, len > 0, v, gs, quad_w);
  }

  // ---- medium runs: the whole warp on one run, group h takes lookups h, h + G, ... ----
  while (medium != 0) {
    const int r = __ffs(medium) - 1;
    medium &= medium - 1;
    const RunView run = view_of(r, __shfl_sync(kFullMask, mine.len, r));
    bool on[kQ];
    typename Quad<WT>::Raw wv[kQ];
#pragma unroll
    for (int k = 0; k < kQ; ++k) {
      on[k] = (v + gs * k) * 4 < run.D;
      wv[k] = Quad<WT>::zero();
      if (on[k] && h == 0) wv[k] = Quad<WT>::load(run.w_lane + k * quad_w);
    }
    float m_old = 0.f;
    if (run.mptr != nullptr) m_old = *run.mptr;
    float4 acc[kQ];
#pragma unroll
    for (int k = 0; k < kQ; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    sum_whole_warp<GT, kScaled, kQ>(p, run, acc, on, gstride_bytes, lane, h, G, gs, quad_g);
    update_row<WT, kQ>(p, run, acc, wv, on, m_old, h == 0, v, gs, quad_w);
  }
}

// One warp per chunk of a long run (kLongRun lookups): the chunk's sum goes to its row of partials.
template <typename KeyT, typename GT, bool kScaled, int kQ>
__global__ void __launch_bounds__(kRunThreads, run_ctas_per_sm<GT>())
    reduce_chunks_groups_kernel(const __grid_constant__ BwdDev p) {
  const int lane = threadIdx.x & 31;
  const int gs = lanes_per_row((p.max_D + 4 * kQ - 1) / (4 * kQ));
  const int gshift = __ffs(gs) - 1;
  const int G = 32 >> gshift;
  const int h = lane >> gshift;
  const int v = lane & (gs - 1);
  const int64_t gstride_bytes = p.grad_stride * static_cast<int64_t>(sizeof(GT));
  const int quad_g = gs * 4 * static_cast<int>(sizeof(GT));
  const int64_t chunks = p.counters[2];
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kRunWarps;
  for (int64_t c = static_cast<int64_t>(blockIdx.x) * kRunWarps + (threadIdx.x >> 5); c < chunks; c += stride) {
    const uint32_t slot = p.chunk_run[c];
    const uint32_t long_id = p.long_run[slot];
    const uint32_t s_run = p.run_start[long_id], e_run = p.run_start[long_id + 1];
    const uint32_t s = s_run + static_cast<uint32_t>(c - p.long_chunk0[slot]) * kLongRun;
    const uint32_t e = s + kLongRun < e_run ? s + kLongRun : e_run;
    const int64_t key = static_cast<int64_t>(reinterpret_cast<const KeyT*>(p.sorted_keys)[s_run]);
    int lo = 0, hi = p.T - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (__ldg(p.hash_size_cumsum + mid) <= key) {
        lo = mid;
      } else {
        hi = mid - 1;
      }
    }
    const int D_begin = __ldg(p.D_offsets + lo);
    RunView run;
    run.len = e - s;
    run.start = s;
    run.pay0 = p.sorted_vals[s];
    run.bag0 = static_cast<uint32_t>(lo) * static_cast<uint32_t>(p.B);
    run.D = __ldg(p.D_offsets + lo + 1) - D_begin;
    run.w_lane = nullptr;
    run.mptr = nullptr;
    run.g_lane = p.grad_output + (p.grad_col_offset + D_begin) * static_cast<int64_t>(sizeof(GT)) +
                 v * 4 * static_cast<int>(sizeof(GT));
    bool on[kQ];
    float4 acc[kQ];
#pragma unroll
    for (int k = 0; k < kQ; ++k) {
      on[k] = (v + gs * k) * 4 < run.D;
      acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    sum_whole_warp<GT, kScaled, kQ>(p, run, acc, on, gstride_bytes, lane, h, G, gs, quad_g);
    float* dst = p.partials + c * p.max_D;
#pragma unroll
    for (int k = 0; k < kQ; ++k)
      if (h == 0 && on[k]) *reinterpret_cast<float4*>(dst + (v + gs * k) * 4) = acc[k];
  }
}
