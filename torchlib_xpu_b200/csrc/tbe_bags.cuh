// One warp per bag, or per group of consecutive bags: the pooled-lookup engine for rows that fit one
// load instruction per lane group.
//
// A plain grid of one-warp CTAs, so that enough independent row loads are in flight to cover HBM /
// L2 latency and the hardware's CTA scheduling balances the load. Measured on B200 this shape beats
// both a persistent variant and the shared-memory ring engine of tbe_stream.cuh. Ids are read 32 at
// a time with one coalesced load and handed out by shuffle as 32-bit row numbers; a row is fetched
// by a group of gs lanes, so one load instruction brings 32/gs rows; loads allocate in L1, where the
// hottest rows of a skewed id stream hit.
// gs = row bytes / 16 rounded up to a power of two (16 for D = 128 fp16); fp16 elements are added to
// the fp32 accumulators with the mixed-precision add of sm_100.
#pragma once
#include "tbe_stream.cuh"

namespace b200tbe {

// One warp per CTA and 32 CTAs per SM (the most an SM holds): a CTA keeps its slot until its longest bag
// is done and bags differ in length by 50 x, so one-warp CTAs keep every slot busy; the 64 registers
// a thread then has pay for eight 16-byte loads in flight per lane. Measured on the 64-table fp16
// step: 3.38 ms, against 3.56 ms for four-warp CTAs with two loads per lane at 64 warps per SM;
// twelve or sixteen loads per lane at 16 CTAs per SM: 5.0 and 6.0 ms.
constexpr int kBagCtasPerSm = 32;
constexpr int kBagLoads = 8;
constexpr uint32_t kNoRow = 0xffffffffu;
// lookups a warp walks in one call at most (positions are 32-bit ints that advance by up to 64)
constexpr int kMaxStream = 0x7fffff00;

// Bags per warp. A warp that walks a group of bags as one stream keeps its load rounds full and reads
// ids ahead, which is worth up to 30 % (64-table fp16 step: 3.36 ms one bag per warp, 2.79 / 2.56 /
// 2.44 / 2.40 ms for groups of 4 / 8 / 16 / 32), as long as the grid still fills the GPU's 148 x 32
// warp slots about five times over (26 tables x 8192 bags: 0.184 ms for groups of 6 to 10, 0.197 for
// 15, 0.221 for 32, 0.211 one bag per warp); a grid smaller than that runs one bag per warp.
inline int bag_group_for(int64_t bags) {
  const int64_t per_slot = bags / (int64_t{kNumSMs} * kBagCtasPerSm * 5);
  return per_slot < 1 ? 1 : (per_slot > 32 ? 32 : static_cast<int>(per_slot));
}

// base + row * row_bytes as one multiply-add (the compiler otherwise spends a multiply and two 64-bit adds).
__device__ __forceinline__ const char* row_address(const char* base, uint32_t row, uint32_t row_bytes) {
  const char* p;
  asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(p) : "r"(row), "r"(row_bytes), "l"(base));
  return p;
}

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

// What a bag kernel knows about its launch, the same for every bag.
template <typename OT>
struct BagLaunch {
  const void* indices;
  const void* offsets;
  const float* per_sample_weights;
  int32_t* status;
  int32_t pooling_mode;
  OT* const* outputs;
  int64_t output_stride;
  int64_t rows_per_dest;
};

// Pools bag `bag` (= t * B + b) of a table of float rows of row_bytes <= 512 bytes, 16-byte aligned,
// and writes it to columns [col, col + D) of sample b.
template <typename WT, typename OT, typename IndexT, bool kWeighted>
__device__ __forceinline__ void pool_float_bag(const BagLaunch<OT>& p, const char* table, int row_bytes,
                                               int64_t num_rows, int64_t col, int64_t bag, int b,
                                               int lane) {
  constexpr int kE = Vec16<WT>::kE;
  constexpr int kLoads = kBagLoads;
  const int64_t start = load_index<IndexT>(p.offsets, bag);
  const int64_t end = load_index<IndexT>(p.offsets, bag + 1);
  const int len = end - start > kMaxStream ? kMaxStream : static_cast<int>(end - start);
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
  // lanes beyond the row's last vector (rows that are not a power of two of vectors) re-read the
  // last one in the test-free rounds; their sums are never stored
  const char* lane_any = table + ((active ? v : vecs - 1) << 4);

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
    // rounds of G * kLoads rows. A round whose rows all exist and are in range -- every round but a
    // bag's last, unless an id is bad -- loads without a test
    const uint32_t bad = __ballot_sync(kFullMask, my_row == kNoRow);   // lanes >= n included
    const int n_clean = bad == 0 ? 32 : __ffs(bad) - 1;                // rows [0, n_clean) are all good
    const int round_rows = G * kLoads;
    int j = 0;
    for (; j + round_rows <= n_clean; j += round_rows) {
      uint4 x[kLoads];
      float w[kLoads];
#pragma unroll
      for (int u = 0; u < kLoads; ++u) {
        const int rr = j + u * G + h;
        const uint32_t row = __shfl_sync(kFullMask, my_row, rr);
        if (kWeighted) w[u] = __shfl_sync(kFullMask, my_w, rr);
        x[u] = ldg_cached16(row_address(lane_any, row, static_cast<uint32_t>(row_bytes)));
      }
#pragma unroll
      for (int u = 0; u < kLoads; ++u) {
        if (kWeighted) {
          Vec16<WT>::fma(acc, x[u], w[u]);
        } else {
          Vec16<WT>::add(acc, x[u]);
        }
      }
    }
    for (; j < n; j += G * kLoads) {
      uint4 x[kLoads];
      float w[kLoads];
#pragma unroll
      for (int u = 0; u < kLoads; ++u) {
        const int rr = j + u * G + h;
        const uint32_t row = __shfl_sync(kFullMask, my_row, rr & 31);
        if (kWeighted) w[u] = __shfl_sync(kFullMask, my_w, rr & 31);
        x[u] = make_uint4(0u, 0u, 0u, 0u);  // +0.0 in either type: adding it changes nothing
        if (rr < n && row != kNoRow && active)
          x[u] = ldg_cached16(row_address(lane_base, row, static_cast<uint32_t>(row_bytes)));
      }
#pragma unroll
      for (int u = 0; u < kLoads; ++u) {
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
    OT* dst = p.outputs[dest] + static_cast<int64_t>(b - dest * rpd) * p.output_stride + col + v * kE;
    float r[kE];
#pragma unroll
    for (int e = 0; e < kE; ++e) r[e] = acc[e] * scale;
#pragma unroll
    for (int e = 0; e < kE; e += 4) store_pooled<OT, 4>(dst + e, r + e);
  }
}

// Pools bags [bag0, bag0 + nb), nb <= 32, of one table (bag0 = t * B + b0) as ONE stream of lookups:
// the bags' ids are consecutive in `indices`, so the warp walks them 32 ids and kLoads load
// instructions at a time whatever the bags' lengths, and closes a bag -- sum over the row groups,
// store -- at the step that holds its last lookup. Against one bag per warp this keeps every load
// round full (a bag of 20 lookups fills 20 of a round's rows) and pays the offsets -> ids -> rows
// latency chain once per group instead of once per bag: the next 32 ids are requested before the
// current ones' rows.
template <typename WT, typename OT, typename IndexT, bool kWeighted>
__device__ __forceinline__ void pool_float_bags(const BagLaunch<OT>& p, const char* table, int row_bytes,
                                                int64_t num_rows, int64_t col, int64_t bag0, int b0, int nb,
                                                int lane) {
  constexpr int kE = Vec16<WT>::kE;
  constexpr int kLoads = kBagLoads;
  // lane i: end of bag i relative to the group's first lookup, made monotone and clamped to 31 bits
  const int64_t begin = load_index<IndexT>(p.offsets, bag0);
  int my_end = 0;
  if (lane < nb) {
    const int64_t e = load_index<IndexT>(p.offsets, bag0 + lane + 1) - begin;
    my_end = e < 0 ? 0 : (e > kMaxStream ? kMaxStream : static_cast<int>(e));
  }
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int below = __shfl_up_sync(kFullMask, my_end, o);
    if (lane >= o && below > my_end) my_end = below;
  }
  const int total = __shfl_sync(kFullMask, my_end, nb - 1);
  const IndexT* idx = reinterpret_cast<const IndexT*>(p.indices) + begin;
  const float* psw = kWeighted ? p.per_sample_weights + begin : nullptr;
  const int vecs = row_bytes >> 4;
  const int gs = lanes_per_row(vecs);
  const int gshift = __ffs(gs) - 1;
  const int G = 32 >> gshift;            // rows per load instruction
  const int h = lane >> gshift;          // this lane's group
  const int v = lane & (gs - 1);         // this lane's vector inside the row
  const bool active = v < vecs;
  const char* lane_base = table + (v << 4);
  // lanes beyond the row's last vector (rows that are not a power of two of vectors) re-read the
  // last one in the test-free rounds; their sums are never stored
  const char* lane_any = table + ((active ? v : vecs - 1) << 4);
  const int64_t row_limit = num_rows >= 0 ? num_rows : int64_t{0xffffffff};
  const bool mean = p.pooling_mode == B200TBE_POOL_MEAN;
  const int rpd = static_cast<int>(p.rows_per_dest);

  float acc[kE];
#pragma unroll
  for (int e = 0; e < kE; ++e) acc[e] = 0.f;
  int cur = 0;                                              // bag being summed (warp-uniform)
  int cur_start = 0;
  int cur_end = __shfl_sync(kFullMask, my_end, 0);

  // where bag `cur` goes: consecutive bags are consecutive rows of a destination
  int dest = b0 / rpd;
  int row_in_dest = b0 - dest * rpd;
  OT* dst = p.outputs[dest] + static_cast<int64_t>(row_in_dest) * p.output_stride + col + v * kE;

  // closes bag `cur`: its sum is spread over the row groups
  auto close_bag = [&]() {
    const int len = cur_end - cur_start;
    const float scale = (mean && len > 0) ? 1.f / static_cast<float>(len) : 1.f;
    if (kE == 8 && gs == 16) {
      // two groups: each keeps half of the lane's elements, so one exchange of four values does it
      float r[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float other = __shfl_xor_sync(kFullMask, h ? acc[e] : acc[e + 4], 16);
        r[e] = ((h ? acc[e + 4] : acc[e]) + other) * scale;
      }
      if (active) store_pooled<OT, 4>(dst + 4 * h, r);
    } else {
      for (int o = gs; o < 32; o <<= 1) {
#pragma unroll
        for (int e = 0; e < kE; ++e) acc[e] += __shfl_xor_sync(kFullMask, acc[e], o);
      }
      if (h == 0 && active) {
        float r[kE];
#pragma unroll
        for (int e = 0; e < kE; ++e) r[e] = acc[e] * scale;
#pragma unroll
        for (int e = 0; e < kE; e += 4) store_pooled<OT, 4>(dst + e, r + e);
      }
    }
#pragma unroll
    for (int e = 0; e < kE; ++e) acc[e] = 0.f;
    ++cur;
    cur_start = cur_end;
    cur_end = __shfl_sync(kFullMask, my_end, cur & 31);
    dst += p.output_stride;
    if (++row_in_dest == rpd && cur < nb) {
      row_in_dest = 0;
      dst = p.outputs[++dest] + col + v * kE;
    }
  };

  IndexT next_id = 0;
  float next_w = 1.f;
  if (lane < total) {
    next_id = __ldg(idx + lane);
    if (kWeighted) next_w = __ldg(psw + lane);
  }
  for (int c = 0; c < total; c += 32) {
    const int n = total - c < 32 ? total - c : 32;
    // this lane's row id; ids do not fit 32 bits only in tables no memory holds
    uint32_t my_row = kNoRow;
    const float my_w = next_w;
    if (lane < n) {
      const int64_t i = static_cast<int64_t>(next_id);
      if (i < 0 || i >= row_limit) {
        if (p.status != nullptr) atomicOr(p.status, B200TBE_DEV_INDEX_OUT_OF_RANGE);
      } else {
        my_row = static_cast<uint32_t>(i);
      }
    }
    if (c + 32 + lane < total) {
      next_id = __ldg(idx + c + 32 + lane);
      if (kWeighted) next_w = __ldg(psw + c + 32 + lane);
    }
    const uint32_t bad = __ballot_sync(kFullMask, my_row == kNoRow);   // lanes >= n included
    const int n_clean = bad == 0 ? 32 : __ffs(bad) - 1;                // rows [0, n_clean) are all good
    const int round_rows = G * kLoads;
    for (int j = 0; j < n; j += round_rows) {
      uint4 x[kLoads];
      float w[kLoads];
      if (j + round_rows <= n_clean) {
        // every row of the round exists and is in range: loads without a test
#pragma unroll
        for (int u = 0; u < kLoads; ++u) {
          const int rr = j + u * G + h;
          const uint32_t row = __shfl_sync(kFullMask, my_row, rr);
          if (kWeighted) w[u] = __shfl_sync(kFullMask, my_w, rr);
          x[u] = ldg_cached16(row_address(lane_any, row, static_cast<uint32_t>(row_bytes)));
        }
      } else {
#pragma unroll
        for (int u = 0; u < kLoads; ++u) {
          const int rr = j + u * G + h;
          const uint32_t row = __shfl_sync(kFullMask, my_row, rr & 31);
          if (kWeighted) w[u] = __shfl_sync(kFullMask, my_w, rr & 31);
          x[u] = make_uint4(0u, 0u, 0u, 0u);  // +0.0 in either type: adding it changes nothing
          if (rr < n && row != kNoRow && active)
            x[u] = ldg_cached16(row_address(lane_base, row, static_cast<uint32_t>(row_bytes)));
        }
      }
      if (c + j + round_rows < cur_end) {        // the whole round inside the open bag, which goes on
#pragma unroll
        for (int u = 0; u < kLoads; ++u) {
          if (kWeighted) {
            Vec16<WT>::fma(acc, x[u], w[u]);
          } else {
            Vec16<WT>::add(acc, x[u]);
          }
        }
        continue;
      }
#pragma unroll
      for (int u = 0; u < kLoads; ++u) {
        const int step = c + j + u * G;          // lookups [step, step + G) of the stream
        if (step + G < cur_end) {                // all of them inside the open bag, which goes on
          if (kWeighted) {
            Vec16<WT>::fma(acc, x[u], w[u]);
          } else {
            Vec16<WT>::add(acc, x[u]);
          }
        } else if (j + u * G < n) {          // (a round of more than 32 rows reaches past the ids at hand)
          // a bag ends in this step: every row goes to the bag that holds it, bags close in order
          const int q = step + h;
          bool pending = true;
          while (cur < nb) {
            if (pending && q < cur_end) {
              if (kWeighted) {
                Vec16<WT>::fma(acc, x[u], w[u]);
              } else {
                Vec16<WT>::add(acc, x[u]);
              }
              pending = false;
            }
            if (step + G < cur_end) break;
            close_bag();
          }
        }
      }
    }
  }
  while (cur < nb) close_bag();   // bags without lookups at the group's end (or a group without any)
}

}  // namespace b200tbe
