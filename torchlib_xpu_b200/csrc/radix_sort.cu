// Stable least-significant-digit radix sort of (key, 32-bit payload) pairs.
//
// One pass per digit of up to 10 bits, three steps per pass, none of which waits on another CTA:
//   1. per-tile digit histograms (shared-memory counters), stored digit-major: counts[d][tile];
//   2. an exclusive scan over that matrix read in storage order, which turns each entry into the
//      global position of the first key of tile `tile` with digit d;
//   3. a scatter: every warp ranks its 32 consecutive keys per round by finding the lanes with an
//      equal digit, one warp vote per digit bit (measured faster than the match instruction; keys
//      of equal digit get consecutive ranks in lane order, so the order of equal keys is kept),
//      the tile is reordered by digit in shared memory, and then written out so that keys of one
//      digit go to consecutive addresses.
// Keys and payloads are read and written exactly once per pass (plus one extra read of the keys
// for the histogram); with 25..28-bit keys that is 3 passes.
//
// Segmented form (SortPlan): the array is a sequence of independent segments (the lookups of one
// embedding table each), every tile lies inside one segment, and the digit counts are stored
// segment-major -- counts[segment][digit][tile of the segment] -- so that ONE exclusive scan over
// the whole matrix still yields global positions, while keys never leave their segment. Only the
// bits that differ inside a segment are sorted: 22 bits for tables of 4 M rows however many tables
// there are.
#include "radix_sort.cuh"
#include "scan.cuh"

namespace b200tbe {
namespace {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kMaxRadix = 2048;        // widest digit table (segmented sort)
constexpr int kDefaultDigitBits = 10;  // widest digit of the unsegmented sort
constexpr int kFlatRadix = 1 << kDefaultDigitBits;
constexpr int kMaxDigitBits = 11;      // widest digit any pass may use

template <typename KeyT>
struct SortTile {
  static constexpr int kItems = sizeof(KeyT) == 4 ? 16 : 8;  // keys per thread
  static constexpr int kTile = kSortThreads * kItems;
};

// Where a CTA's tile lies and where its digit counts go. Flat sort: tile i is keys
// [i * kTile, ...), counts[d * num_tiles + i]. Segmented sort: read from the tile's descriptor.
struct TilePlace {
  int64_t base;
  int tile_n;
  int64_t col;     // index of digit 0's count
  int64_t stride;  // distance between consecutive digits' counts
  bool live;
};

template <int kTile>
__device__ __forceinline__ TilePlace place_tile(int64_t n, int radix, int num_tiles, const uint4* desc,
                                                const uint32_t* seg_tile_base,
                                                const uint32_t* total_tiles) {
  TilePlace t;
  if (desc == nullptr) {
    t.base = static_cast<int64_t>(blockIdx.x) * kTile;
    t.tile_n = n - t.base < kTile ? static_cast<int>(n - t.base) : kTile;
    t.col = blockIdx.x;
    t.stride = num_tiles;
    t.live = true;
    return t;
  }
  t.live = blockIdx.x < __ldg(total_tiles);
  if (!t.live) return t;
  const uint4 d = __ldg(desc + blockIdx.x);  // {begin, count, segment, first tile of the segment}
  t.base = d.x;
  t.tile_n = static_cast<int>(d.y);
  t.stride = __ldg(seg_tile_base + d.z + 1) - d.w;
  t.col = static_cast<int64_t>(radix) * d.w + (blockIdx.x - d.w);
  return t;
}

template <typename KeyT>
__global__ void __launch_bounds__(kSortThreads)
    sort_histogram_kernel(const KeyT* __restrict__ keys, int64_t n, int shift, uint32_t mask,
                          int radix, uint32_t* __restrict__ counts, int num_tiles,
                          const uint4* __restrict__ desc, const uint32_t* __restrict__ seg_tile_base,
                          const uint32_t* __restrict__ total_tiles) {
  constexpr int kItems = SortTile<KeyT>::kItems;
  constexpr int kTile = SortTile<KeyT>::kTile;
  __shared__ uint32_t hist[kMaxRadix];
  const TilePlace tp = place_tile<kTile>(n, radix, num_tiles, desc, seg_tile_base, total_tiles);
  if (!tp.live) return;
  // all of the thread's keys are requested before the first is counted
  KeyT k[kItems];
#pragma unroll
  for (int i = 0; i < kItems; ++i) {
    const int it = i * kSortThreads + threadIdx.x;
    k[i] = it < tp.tile_n ? keys[tp.base + it] : KeyT(0);
  }
  for (int d = threadIdx.x; d < radix; d += kSortThreads) hist[d] = 0;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kItems; ++i) {
    const int it = i * kSortThreads + threadIdx.x;
    if (it < tp.tile_n) atomicAdd(&hist[static_cast<uint32_t>(k[i] >> shift) & mask], 1u);
  }
  __syncthreads();
  for (int d = threadIdx.x; d < radix; d += kSortThreads) counts[d * tp.stride + tp.col] = hist[d];
}

// Shared memory of the scatter kernel: per-warp digit counters (16 bits are enough: a warp holds
// at most 32 * kItems keys, a tile at most 4096), the tile-level digit offsets, and the staging
// area in which the tile is reordered. Once the tile is staged the counters are dead and their
// space holds the per-digit distance from staging position to global position. For 4-byte keys:
// 38 KB with 256 digits (five CTAs per SM at 48 registers: 0.5 % faster than four at 64), 52 KB
// with 1024 (four), 72 KB with 2048 (three).
template <typename KeyT, int kRadix>
struct ScatterSmem {
  union {
    uint16_t warp_hist[kSortWarps][kRadix];
    uint32_t delta[kRadix];
  };
  uint32_t digit_start[kRadix];
  KeyT keys[SortTile<KeyT>::kTile];
  uint32_t vals[SortTile<KeyT>::kTile];
};

// kRadix: capacity of the digit tables (>= radix, a multiple of kSortThreads). kFull: the tile holds
// kTile keys (every tile but a segment's last), so no step tests a position against the tile's end.
template <typename KeyT, int kRadix, bool kFull>
__device__ __forceinline__ void scatter_tile(ScatterSmem<KeyT, kRadix>& sm, const TilePlace& tp,
                                             const KeyT* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                                             KeyT* __restrict__ keys_out, uint32_t* __restrict__ vals_out,
                                             int shift, uint32_t mask, int radix,
                                             const uint32_t* __restrict__ positions) {
  constexpr int kItems = SortTile<KeyT>::kItems;
  constexpr int kTile = SortTile<KeyT>::kTile;
  constexpr int kDigitsPerThread = kRadix / kSortThreads;
  constexpr int kBits = kRadix == 256 ? 8 : (kRadix == 1024 ? 10 : 11);   // bits above the pass's digit are zero
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  {
    uint32_t* z = reinterpret_cast<uint32_t*>(&sm.warp_hist[0][0]);
    for (int i = threadIdx.x; i < kSortWarps * kRadix / 2; i += kSortThreads) z[i] = 0;
  }

  const int64_t base = tp.base;
  const int tile_n = kFull ? kTile : tp.tile_n;
  const int warp_base = warp * (kItems * 32);
  const uint32_t lanemask_lt = (1u << lane) - 1u;

  // all of the thread's keys are requested before the first is looked at
  KeyT k[kItems];
#pragma unroll
  for (int r = 0; r < kItems; ++r) {
    const int it = warp_base + r * 32 + lane;
    k[r] = (kFull || it < tile_n) ? keys_in[base + it] : KeyT(0);
  }
  __syncthreads();

  uint32_t rank[kItems];
#pragma unroll
  for (int r = 0; r < kItems; ++r) {
    const int it = warp_base + r * 32 + lane;
    const bool valid = kFull || it < tile_n;
    rank[r] = 0;
    const uint32_t d = static_cast<uint32_t>(k[r] >> shift) & mask;
    // lanes holding the same digit, found one bit at a time with warp votes
    uint32_t peers = kFull ? kFullMask : __ballot_sync(kFullMask, valid);
#pragma unroll
    for (int b = 0; b < kBits; ++b) {
      const bool bit = (d >> b) & 1u;
      const uint32_t with_bit = __ballot_sync(kFullMask, bit);
      peers &= bit ? with_bit : ~with_bit;
    }
    if (valid) {
      const int leader = __ffs(peers) - 1;
      uint32_t before = 0;
      if (lane == leader) {
        before = sm.warp_hist[warp][d];
        sm.warp_hist[warp][d] = static_cast<uint16_t>(before + __popc(peers));
      }
      before = __shfl_sync(peers, before, leader);
      rank[r] = before + __popc(peers & lanemask_lt);
    }
    __syncwarp();
  }
  __syncthreads();

  // per digit: exclusive prefix over the warps, then over the digits of the tile; thread i owns
  // the kDigitsPerThread consecutive digits starting at i * kDigitsPerThread
  uint32_t totals[kDigitsPerThread], run_total[kDigitsPerThread];
  uint32_t thread_total = 0;
#pragma unroll
  for (int j = 0; j < kDigitsPerThread; ++j) {
    const int d = threadIdx.x * kDigitsPerThread + j;
    uint32_t run = 0;
#pragma unroll
    for (int w = 0; w < kSortWarps; ++w) {
      const uint32_t c = sm.warp_hist[w][d];
      sm.warp_hist[w][d] = static_cast<uint16_t>(run);
      run += c;
    }
    run_total[j] = run;
    thread_total += run;
  }
  uint32_t unused_total;
  uint32_t start = block_exclusive_scan(thread_total, &unused_total);
#pragma unroll
  for (int j = 0; j < kDigitsPerThread; ++j) {
    const int d = threadIdx.x * kDigitsPerThread + j;
    sm.digit_start[d] = start;
    // global position of the tile's first key of digit d, minus its staging position
    totals[j] = (d < radix ? positions[d * tp.stride + tp.col] : 0u) - start;
    start += run_total[j];
  }
  __syncthreads();

#pragma unroll
  for (int r = 0; r < kItems; ++r) {
    const int it = warp_base + r * 32 + lane;
    if (kFull || it < tile_n) {
      const uint32_t d = static_cast<uint32_t>(k[r] >> shift) & mask;
      const uint32_t pos = sm.digit_start[d] + sm.warp_hist[warp][d] + rank[r];
      sm.keys[pos] = k[r];
      sm.vals[pos] = vals_in[base + it];
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kDigitsPerThread; ++j) sm.delta[threadIdx.x * kDigitsPerThread + j] = totals[j];
  __syncthreads();

  if (kFull) {
#pragma unroll 4
    for (int i = threadIdx.x; i < kTile; i += kSortThreads) {
      const KeyT key = sm.keys[i];
      const uint32_t d = static_cast<uint32_t>(key >> shift) & mask;
      const uint32_t dst = static_cast<uint32_t>(i) + sm.delta[d];
      keys_out[dst] = key;
      vals_out[dst] = sm.vals[i];
    }
  } else {
    for (int i = threadIdx.x; i < tile_n; i += kSortThreads) {
      const KeyT key = sm.keys[i];
      const uint32_t d = static_cast<uint32_t>(key >> shift) & mask;
      const uint32_t dst = static_cast<uint32_t>(i) + sm.delta[d];
      keys_out[dst] = key;
      vals_out[dst] = sm.vals[i];
    }
  }
}

template <typename KeyT, int kRadix>
__global__ void __launch_bounds__(kSortThreads, kRadix > 1024 ? 3 : (kRadix > 256 ? 4 : 5))
    sort_scatter_kernel(const KeyT* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                        KeyT* __restrict__ keys_out, uint32_t* __restrict__ vals_out, int64_t n,
                        int shift, uint32_t mask, int radix,
                        const uint32_t* __restrict__ positions, int num_tiles,
                        const uint4* __restrict__ desc, const uint32_t* __restrict__ seg_tile_base,
                        const uint32_t* __restrict__ total_tiles) {
  constexpr int kTile = SortTile<KeyT>::kTile;
  extern __shared__ __align__(16) unsigned char sort_smem[];
  ScatterSmem<KeyT, kRadix>& sm = *reinterpret_cast<ScatterSmem<KeyT, kRadix>*>(sort_smem);
  const TilePlace tp = place_tile<kTile>(n, radix, num_tiles, desc, seg_tile_base, total_tiles);
  if (!tp.live) return;
  if (tp.tile_n == kTile) {
    scatter_tile<KeyT, kRadix, true>(sm, tp, keys_in, vals_in, keys_out, vals_out, shift, mask, radix, positions);
  } else {
    scatter_tile<KeyT, kRadix, false>(sm, tp, keys_in, vals_in, keys_out, vals_out, shift, mask, radix, positions);
  }
}

// ---- plan of a segmented sort -------------------------------------------------------------------
// seg_start[s] = offsets[s * stride] (clamped to n), seg_tile_base = exclusive prefix of the tiles
// per segment. One CTA.
__global__ void __launch_bounds__(kScanThreads)
    plan_segments_kernel(const void* __restrict__ offsets, int offset_bytes, int num_segments, int64_t stride,
                         int64_t n, int max_tiles, uint32_t* __restrict__ seg_start,
                         uint32_t* __restrict__ seg_tile_base, uint32_t* __restrict__ total_tiles,
                         int32_t* status) {
  uint32_t carry = 0;
  auto start_of = [&](int s) -> int64_t {
    const int64_t i = static_cast<int64_t>(s) * stride;
    int64_t v = offset_bytes == 8 ? load_index<int64_t>(offsets, i) : load_index<int32_t>(offsets, i);
    if (v < 0) v = 0;
    return v > n ? n : v;
  };
  for (int base = 0; base <= num_segments; base += kScanThreads) {
    const int s = base + threadIdx.x;
    uint32_t tiles = 0;
    if (s <= num_segments) {
      const int64_t first = start_of(s);
      seg_start[s] = static_cast<uint32_t>(first);
      if (s < num_segments) {
        const int64_t len = start_of(s + 1) - first;
        tiles = len > 0 ? static_cast<uint32_t>((len + kSortPlanTile - 1) / kSortPlanTile) : 0u;
      }
    }
    uint32_t total;
    const uint32_t prefix = block_exclusive_scan(tiles, &total);
    if (s <= num_segments) seg_tile_base[s] = carry + prefix;
    carry += total;
  }
  if (threadIdx.x == 0) {
    if (carry > static_cast<uint32_t>(max_tiles)) {   // offsets that do not describe n keys
      if (status != nullptr) atomicOr(status, B200TBE_DEV_OFFSETS_NOT_MONOTONE);
      carry = static_cast<uint32_t>(max_tiles);
    }
    *total_tiles = carry;
  }
}

__global__ void __launch_bounds__(256)
    plan_tiles_kernel(const uint32_t* __restrict__ seg_start, const uint32_t* __restrict__ seg_tile_base,
                      int num_segments, const uint32_t* __restrict__ total_tiles,
                      uint4* __restrict__ tile_desc) {
  const uint32_t tile = blockIdx.x * blockDim.x + threadIdx.x;
  if (tile >= *total_tiles) return;
  // the last segment whose first tile is <= tile (empty segments share their successor's value)
  int lo = 0, hi = num_segments - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (__ldg(seg_tile_base + mid) <= tile) {
      lo = mid;
    } else {
      hi = mid - 1;
    }
  }
  const uint32_t first = __ldg(seg_tile_base + lo);
  const uint32_t begin = __ldg(seg_start + lo) + (tile - first) * kSortPlanTile;
  const uint32_t end = __ldg(seg_start + lo + 1);
  const uint32_t count = end - begin < static_cast<uint32_t>(kSortPlanTile) ? end - begin : kSortPlanTile;
  tile_desc[tile] = make_uint4(begin, count, static_cast<uint32_t>(lo), first);
}

template <typename KeyT>
int64_t sort_num_tiles(int64_t n) {
  return (n + SortTile<KeyT>::kTile - 1) / SortTile<KeyT>::kTile;
}

struct PassArgs {
  int64_t n;
  int shift, bits, tiles;
  uint32_t* counts;
  const SortPlan* plan;
};

template <typename KeyT, int kRadix>
int launch_scatter(const KeyT* kin, const uint32_t* vin, KeyT* kout, uint32_t* vout, const PassArgs& a,
                   cudaStream_t stream) {
  auto kernel = sort_scatter_kernel<KeyT, kRadix>;
  const size_t smem = sizeof(ScatterSmem<KeyT, kRadix>);
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return B200TBE_ERR_LAUNCH;
  const int radix = 1 << a.bits;
  kernel<<<a.tiles, kSortThreads, smem, stream>>>(
      kin, vin, kout, vout, a.n, a.shift, static_cast<uint32_t>(radix - 1), radix, a.counts,
      a.tiles, a.plan ? a.plan->tile_desc : nullptr, a.plan ? a.plan->seg_tile_base : nullptr,
      a.plan ? a.plan->total_tiles : nullptr);
  return B200TBE_OK;
}

// plan == nullptr: one flat array of n keys. Otherwise the tiles of the plan (tiles = its bound).
template <typename KeyT>
int sort_impl(KeyT* keys_a, uint32_t* vals_a, KeyT* keys_b, uint32_t* vals_b, int64_t n,
              int key_bits, int max_digit_bits, const SortPlan* plan, uint32_t* counts,
              uint32_t* tile_sums, bool* result_in_b, cudaStream_t stream) {
  const int64_t tiles64 = plan ? plan->max_tiles : sort_num_tiles<KeyT>(n);
  if (tiles64 > 0x7fffffff / (plan ? kMaxRadix : kFlatRadix)) return B200TBE_ERR_TOO_LARGE;
  const int tiles = static_cast<int>(tiles64);
  const int passes = (key_bits + max_digit_bits - 1) / max_digit_bits;
  bool in_b = false;
  int shift = 0;
  for (int pass = 0; pass < passes; ++pass) {
    // spread the bits evenly: fewer bins per pass means cheaper ranking
    const int bits = (key_bits - shift + (passes - pass) - 1) / (passes - pass);
    const int radix = 1 << bits;
    const uint32_t mask = static_cast<uint32_t>(radix - 1);
    const KeyT* kin = in_b ? keys_b : keys_a;
    const uint32_t* vin = in_b ? vals_b : vals_a;
    KeyT* kout = in_b ? keys_a : keys_b;
    uint32_t* vout = in_b ? vals_a : vals_b;
    sort_histogram_kernel<KeyT><<<tiles, kSortThreads, 0, stream>>>(
        kin, n, shift, mask, radix, counts, tiles, plan ? plan->tile_desc : nullptr,
        plan ? plan->seg_tile_base : nullptr, plan ? plan->total_tiles : nullptr);
    // with a plan the scan also covers the unused tail of the matrix (tiles is an upper bound);
    // nothing reads it
    int st = exclusive_scan_u32(counts, static_cast<int64_t>(radix) * tiles, tile_sums, nullptr, stream);
    if (st != B200TBE_OK) return st;
    const PassArgs a{n, shift, bits, tiles, counts, plan};
    if (bits <= 8) {
      st = launch_scatter<KeyT, 256>(kin, vin, kout, vout, a, stream);
    } else if (bits <= 10) {
      st = launch_scatter<KeyT, 1024>(kin, vin, kout, vout, a, stream);
    } else {
      st = launch_scatter<KeyT, 2048>(kin, vin, kout, vout, a, stream);
    }
    if (st != B200TBE_OK) return st;
    in_b = !in_b;
    shift += bits;
  }
  *result_in_b = in_b;
  return launch_status();
}

size_t align256(size_t x) { return (x + 255) & ~size_t{255}; }

}  // namespace

size_t radix_sort_scratch_bytes(int64_t n) {
  if (n <= 0) return 256;
  // tile count of the narrower tile (8-byte keys) bounds both key widths
  const int64_t tiles = sort_num_tiles<uint64_t>(n);
  const int64_t counts = tiles * kFlatRadix;
  return align256(static_cast<size_t>(counts) * 4) +
         align256(static_cast<size_t>(scan_num_tiles(counts)) * 4) + 256;
}

size_t radix_sort_planned_scratch_bytes(int64_t max_tiles) {
  const int64_t counts = (max_tiles > 0 ? max_tiles : 1) * kMaxRadix;
  return align256(static_cast<size_t>(counts) * 4) +
         align256(static_cast<size_t>(scan_num_tiles(counts)) * 4) + 256;
}

int64_t sort_plan_max_tiles(int64_t n, int64_t num_segments) {
  // every segment's last tile may be partial
  return n / kSortPlanTile + (num_segments > 0 ? num_segments : 0) + 1;
}

size_t sort_plan_bytes(int64_t n, int64_t num_segments) {
  const int64_t tiles = sort_plan_max_tiles(n, num_segments);
  return 2 * align256(static_cast<size_t>(num_segments + 1) * 4) + align256(static_cast<size_t>(tiles) * sizeof(uint4)) + 256;
}

int build_sort_plan(const void* offsets, int offset_bytes, int num_segments, int64_t stride, int64_t n,
                    void* plan_mem, int32_t* status, SortPlan* plan, const uint32_t** seg_start_out,
                    cudaStream_t stream) {
  const int64_t tiles = sort_plan_max_tiles(n, num_segments);
  if (tiles > 0x7fffffff / kMaxRadix || num_segments < 1) return B200TBE_ERR_TOO_LARGE;
  char* at = static_cast<char*>(plan_mem);
  uint32_t* seg_start = reinterpret_cast<uint32_t*>(at);
  at += align256(static_cast<size_t>(num_segments + 1) * 4);
  uint32_t* seg_tile_base = reinterpret_cast<uint32_t*>(at);
  at += align256(static_cast<size_t>(num_segments + 1) * 4);
  uint4* tile_desc = reinterpret_cast<uint4*>(at);
  at += align256(static_cast<size_t>(tiles) * sizeof(uint4));
  uint32_t* total_tiles = reinterpret_cast<uint32_t*>(at);
  plan_segments_kernel<<<1, kScanThreads, 0, stream>>>(offsets, offset_bytes, num_segments, stride, n,
                                                      static_cast<int>(tiles), seg_start, seg_tile_base,
                                                      total_tiles, status);
  plan_tiles_kernel<<<static_cast<unsigned>((tiles + 255) / 256), 256, 0, stream>>>(
      seg_start, seg_tile_base, num_segments, total_tiles, tile_desc);
  plan->tile_desc = tile_desc;
  plan->seg_tile_base = seg_tile_base;
  plan->total_tiles = total_tiles;
  plan->max_tiles = static_cast<int>(tiles);
  if (seg_start_out != nullptr) *seg_start_out = seg_start;
  return launch_status();
}

int radix_sort_pairs_planned(uint32_t* keys_a, uint32_t* vals_a, uint32_t* keys_b, uint32_t* vals_b,
                             int64_t n, int key_bits, int max_digit_bits, const SortPlan& plan,
                             void* scratch, size_t scratch_bytes, bool* result_in_b,
                             cudaStream_t stream) {
  *result_in_b = false;
  if (n < 0 || key_bits < 0 || key_bits > 32 || max_digit_bits < 1 || max_digit_bits > kMaxDigitBits ||
      plan.max_tiles < 0)
    return B200TBE_ERR_BAD_ARG;
  if (n == 0 || key_bits == 0 || plan.max_tiles == 0) return B200TBE_OK;
  if (scratch == nullptr || scratch_bytes < radix_sort_planned_scratch_bytes(plan.max_tiles) ||
      !aligned_to(scratch, 256))
    return B200TBE_ERR_SCRATCH;
  uint32_t* counts = static_cast<uint32_t*>(scratch);
  uint32_t* tile_sums = reinterpret_cast<uint32_t*>(
      static_cast<char*>(scratch) + align256(static_cast<size_t>(plan.max_tiles) * kMaxRadix * 4));
  return sort_impl<uint32_t>(keys_a, vals_a, keys_b, vals_b, n, key_bits, max_digit_bits, &plan, counts,
                             tile_sums, result_in_b, stream);
}

int radix_sort_pairs(void* keys_a, uint32_t* vals_a, void* keys_b, uint32_t* vals_b, int64_t n,
                     int key_bytes, int key_bits, void* scratch, size_t scratch_bytes,
                     bool* result_in_b, cudaStream_t stream) {
  *result_in_b = false;
  if (n < 0 || key_bits < 0 || (key_bytes != 4 && key_bytes != 8) || key_bits > key_bytes * 8)
    return B200TBE_ERR_BAD_ARG;
  if (n >= (int64_t{1} << 31)) return B200TBE_ERR_TOO_LARGE;
  if (n == 0 || key_bits == 0) return B200TBE_OK;
  if (keys_a == nullptr || vals_a == nullptr || keys_b == nullptr || vals_b == nullptr)
    return B200TBE_ERR_BAD_ARG;
  if (scratch == nullptr || scratch_bytes < radix_sort_scratch_bytes(n) ||
      !aligned_to(scratch, 256))
    return B200TBE_ERR_SCRATCH;
  const int64_t tiles = sort_num_tiles<uint64_t>(n);
  uint32_t* counts = static_cast<uint32_t*>(scratch);
  uint32_t* tile_sums = reinterpret_cast<uint32_t*>(
      static_cast<char*>(scratch) + align256(static_cast<size_t>(tiles) * kFlatRadix * 4));
  if (key_bytes == 4)
    return sort_impl<uint32_t>(static_cast<uint32_t*>(keys_a), vals_a,
                               static_cast<uint32_t*>(keys_b), vals_b, n, key_bits,
                               kDefaultDigitBits, nullptr, counts, tile_sums, result_in_b, stream);
  return sort_impl<unsigned long long>(static_cast<unsigned long long*>(keys_a), vals_a,
                                       static_cast<unsigned long long*>(keys_b), vals_b, n, key_bits,
                                       kDefaultDigitBits, nullptr, counts, tile_sums, result_in_b,
                                       stream);
}

}  // namespace b200tbe

using namespace b200tbe;

extern "C" size_t b200tbe_radix_sort_scratch_bytes(int64_t n) { return radix_sort_scratch_bytes(n); }

extern "C" int b200tbe_radix_sort_pairs(void* keys_in, uint32_t* vals_in, void* keys_out,
                                        uint32_t* vals_out, int64_t n, int32_t key_bytes,
                                        int32_t key_bits, void* scratch, size_t scratch_bytes,
                                        b200tbe_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  bool in_b = false;
  const int st = radix_sort_pairs(keys_in, vals_in, keys_out, vals_out, n, key_bytes, key_bits,
                                  scratch, scratch_bytes, &in_b, stream);
  if (st != B200TBE_OK || n <= 0) return st;
  if (!in_b) {
    if (cudaMemcpyAsync(keys_out, keys_in, static_cast<size_t>(n) * key_bytes,
                        cudaMemcpyDeviceToDevice, stream) != cudaSuccess ||
        cudaMemcpyAsync(vals_out, vals_in, static_cast<size_t>(n) * 4, cudaMemcpyDeviceToDevice,
                        stream) != cudaSuccess)
      return B200TBE_ERR_LAUNCH;
  }
  return B200TBE_OK;
}

extern "C" size_t b200tbe_radix_sort_segments_scratch_bytes(int64_t n, int32_t num_segments) {
  if (n < 0 || num_segments < 0) return 0;
  return sort_plan_bytes(n, num_segments) +
         radix_sort_planned_scratch_bytes(sort_plan_max_tiles(n, num_segments));
}

extern "C" int b200tbe_radix_sort_segments(uint32_t* keys_in, uint32_t* vals_in, uint32_t* keys_out,
                                           uint32_t* vals_out, int64_t n, const void* seg_offsets,
                                           int32_t offset_bytes, int32_t num_segments, int32_t key_bits,
                                           void* scratch, size_t scratch_bytes, b200tbe_stream_t stream_) {
  if (n < 0 || num_segments < 0 || key_bits < 0 || key_bits > 32 || (offset_bytes != 4 && offset_bytes != 8))
    return B200TBE_ERR_BAD_ARG;
  if (n >= (int64_t{1} << 31)) return B200TBE_ERR_TOO_LARGE;
  if (n == 0 || num_segments == 0) return B200TBE_OK;
  if (keys_in == nullptr || vals_in == nullptr || keys_out == nullptr || vals_out == nullptr ||
      seg_offsets == nullptr)
    return B200TBE_ERR_BAD_ARG;
  if (scratch == nullptr || scratch_bytes < b200tbe_radix_sort_segments_scratch_bytes(n, num_segments) ||
      !aligned_to(scratch, 256))
    return B200TBE_ERR_SCRATCH;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  SortPlan plan{};
  int st = build_sort_plan(seg_offsets, offset_bytes, num_segments, 1, n, scratch, nullptr, &plan, nullptr,
                           stream);
  if (st != B200TBE_OK) return st;
  char* sort_scratch = static_cast<char*>(scratch) + sort_plan_bytes(n, num_segments);
  bool in_b = false;
  st = radix_sort_pairs_planned(keys_in, vals_in, keys_out, vals_out, n, key_bits, kMaxDigitBits, plan,
                                sort_scratch, radix_sort_planned_scratch_bytes(plan.max_tiles), &in_b,
                                stream);
  if (st != B200TBE_OK) return st;
  if (!in_b) {
    if (cudaMemcpyAsync(keys_out, keys_in, static_cast<size_t>(n) * 4, cudaMemcpyDeviceToDevice, stream) !=
            cudaSuccess ||
        cudaMemcpyAsync(vals_out, vals_in, static_cast<size_t>(n) * 4, cudaMemcpyDeviceToDevice, stream) !=
            cudaSuccess)
      return B200TBE_ERR_LAUNCH;
  }
  return B200TBE_OK;
}

// ------------------------------------------------------------------------------------------------
// Sort entry point that allocates nothing.
//
// Some callers of this library cannot obtain device memory at call time: a C or C++ host that links
// libb200tbe.so directly and has no tensor allocator to borrow scratch from; a serving process that
// reserves all of HBM for embedding tables at start-up, so a later cudaMalloc may fail; and
// latency-critical loops that cannot afford the device-wide synchronisation cudaMalloc and cudaFree
// imply. For them the sort's scratch (per-tile digit counts and the scan's tile sums) lives in a
// fixed array inside the library. Every GPU that loads the library holds the array until the
// process exits, which is why the capacity is modest.
// ------------------------------------------------------------------------------------------------
namespace b200tbe {
namespace {

constexpr int64_t kStaticSortMaxPairs = int64_t{1} << 20;
// counts for the narrower (8-byte-key) tile + scan tile sums + slack, as radix_sort_scratch_bytes()
// computes for kStaticSortMaxPairs: 512 tiles x 1024 digits x 4 B = 2 MiB, plus under 4 KiB.
constexpr size_t kStaticSortScratchBytes = (size_t{512} * kFlatRadix * 4) + 4096;

static __device__ __align__(256) unsigned char g_static_sort_scratch[kStaticSortScratchBytes];

constexpr int kMaxDevices = 64;
void* g_static_sort_ptr[kMaxDevices] = {};

// The array's name is only a host-side handle; the device address has to be asked for, once per
// device, with that device current.
int static_sort_scratch(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200TBE_ERR_LAUNCH;
  void* p = __atomic_load_n(&g_static_sort_ptr[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    if (cudaGetSymbolAddress(&p, g_static_sort_scratch) != cudaSuccess || p == nullptr)
      return B200TBE_ERR_LAUNCH;
    __atomic_store_n(&g_static_sort_ptr[dev], p, __ATOMIC_RELEASE);
  }
  *out = p;
  return B200TBE_OK;
}

}  // namespace
}  // namespace b200tbe

extern "C" int64_t b200tbe_radix_sort_pairs_static_max(void) { return kStaticSortMaxPairs; }

extern "C" int b200tbe_radix_sort_pairs_static(void* keys_in, uint32_t* vals_in, void* keys_out,
                                               uint32_t* vals_out, int64_t n, int32_t key_bytes,
                                               int32_t key_bits, b200tbe_stream_t stream_) {
  if (n < 0) return B200TBE_ERR_BAD_ARG;
  if (n > kStaticSortMaxPairs) return B200TBE_ERR_TOO_LARGE;
  static_assert(kStaticSortScratchBytes >= 256, "scratch too small");
  if (radix_sort_scratch_bytes(n) > kStaticSortScratchBytes) return B200TBE_ERR_TOO_LARGE;
  void* scratch = nullptr;
  const int st = static_sort_scratch(&scratch);
  if (st != B200TBE_OK) return st;
  // Nothing in the scratch has to start at zero: every pass rewrites all the counts it reads.
  return b200tbe_radix_sort_pairs(keys_in, vals_in, keys_out, vals_out, n, key_bytes, key_bits,
                                  scratch, kStaticSortScratchBytes, stream_);
}
