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
#include "radix_sort.cuh"
#include "scan.cuh"

namespace b200tbe {
namespace {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kMaxRadix = 1024;
constexpr int kDigitsPerThread = kMaxRadix / kSortThreads;
constexpr int kMaxDigitBits = 10;

template <typename KeyT>
struct SortTile {
  static constexpr int kItems = sizeof(KeyT) == 4 ? 16 : 8;  // keys per thread
  static constexpr int kTile = kSortThreads * kItems;
};

template <typename KeyT>
__global__ void __launch_bounds__(kSortThreads)
    sort_histogram_kernel(const KeyT* __restrict__ keys, int64_t n, int shift, uint32_t mask,
                          int radix, uint32_t* __restrict__ counts, int num_tiles) {
  constexpr int kItems = SortTile<KeyT>::kItems;
  constexpr int kTile = SortTile<KeyT>::kTile;
  __shared__ uint32_t hist[kMaxRadix];
  for (int d = threadIdx.x; d < kMaxRadix; d += kSortThreads) hist[d] = 0;
  __syncthreads();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kTile;
#pragma unroll
  for (int i = 0; i < kItems; ++i) {
    const int64_t idx = base + i * kSortThreads + threadIdx.x;
    if (idx < n) atomicAdd(&hist[static_cast<uint32_t>(keys[idx] >> shift) & mask], 1u);
  }
  __syncthreads();
  for (int d = threadIdx.x; d < radix; d += kSortThreads)
    counts[static_cast<int64_t>(d) * num_tiles + blockIdx.x] = hist[d];
}

// Shared memory of the scatter kernel: per-warp digit counters (16 bits are enough: a warp holds
// at most 32 * kItems keys, a tile at most 4096), the tile-level digit offsets, and the staging
// area in which the tile is reordered. Once the tile is staged the counters are dead and their
// space holds the per-digit distance from staging position to global position. 52 KB for 4-byte
// keys: four CTAs per SM.
template <typename KeyT>
struct ScatterSmem {
  union {
    uint16_t warp_hist[kSortWarps][kMaxRadix];
    uint32_t delta[kMaxRadix];
  };
  uint32_t digit_start[kMaxRadix];
  KeyT keys[SortTile<KeyT>::kTile];
  uint32_t vals[SortTile<KeyT>::kTile];
};

template <typename KeyT>
__global__ void __launch_bounds__(kSortThreads, 4)
    sort_scatter_kernel(const KeyT* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                        KeyT* __restrict__ keys_out, uint32_t* __restrict__ vals_out, int64_t n,
                        int shift, uint32_t mask, int radix, int digit_bits,
                        const uint32_t* __restrict__ positions, int num_tiles) {
  constexpr int kItems = SortTile<KeyT>::kItems;
  constexpr int kTile = SortTile<KeyT>::kTile;
  extern __shared__ __align__(16) unsigned char sort_smem[];
  ScatterSmem<KeyT>& sm = *reinterpret_cast<ScatterSmem<KeyT>*>(sort_smem);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  {
    uint32_t* z = reinterpret_cast<uint32_t*>(&sm.warp_hist[0][0]);
    for (int i = threadIdx.x; i < kSortWarps * kMaxRadix / 2; i += kSortThreads) z[i] = 0;
  }

  const int64_t base = static_cast<int64_t>(blockIdx.x) * kTile;
  const int tile_n = n - base < kTile ? static_cast<int>(n - base) : kTile;
  const int warp_base = warp * (kItems * 32);
  const uint32_t lanemask_lt = (1u << lane) - 1u;

  // all of the thread's keys are requested before the first is looked at
  KeyT k[kItems];
#pragma unroll
  for (int r = 0; r < kItems; ++r) {
    const int it = warp_base + r * 32 + lane;
    k[r] = it < tile_n ? keys_in[base + it] : KeyT(0);
  }
  __syncthreads();

  uint32_t rank[kItems];
#pragma unroll
  for (int r = 0; r < kItems; ++r) {
    const int it = warp_base + r * 32 + lane;
    const bool valid = it < tile_n;
    rank[r] = 0;
    const uint32_t d = static_cast<uint32_t>(k[r] >> shift) & mask;
    // lanes holding the same digit, found one bit at a time with warp votes
    uint32_t peers = __ballot_sync(kFullMask, valid);
    for (int b = 0; b < digit_bits; ++b) {
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
    totals[j] = (d < radix ? positions[static_cast<int64_t>(d) * num_tiles + blockIdx.x] : 0u) - start;
    start += run_total[j];
  }
  __syncthreads();

#pragma unroll
  for (int r = 0; r < kItems; ++r) {
    const int it = warp_base + r * 32 + lane;
    if (it < tile_n) {
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

  for (int i = threadIdx.x; i < tile_n; i += kSortThreads) {
    const KeyT key = sm.keys[i];
    const uint32_t d = static_cast<uint32_t>(key >> shift) & mask;
    const uint32_t dst = static_cast<uint32_t>(i) + sm.delta[d];
    keys_out[dst] = key;
    vals_out[dst] = sm.vals[i];
  }
}

template <typename KeyT>
int64_t sort_num_tiles(int64_t n) {
  return (n + SortTile<KeyT>::kTile - 1) / SortTile<KeyT>::kTile;
}

template <typename KeyT>
int sort_impl(KeyT* keys_a, uint32_t* vals_a, KeyT* keys_b, uint32_t* vals_b, int64_t n,
              int key_bits, uint32_t* counts, uint32_t* tile_sums, bool* result_in_b,
              cudaStream_t stream) {
  const int64_t tiles64 = sort_num_tiles<KeyT>(n);
  if (tiles64 > 0x7fffffff / kMaxRadix) return B200TBE_ERR_TOO_LARGE;
  const int tiles = static_cast<int>(tiles64);
  const int passes = (key_bits + kMaxDigitBits - 1) / kMaxDigitBits;
  const size_t scatter_smem = sizeof(ScatterSmem<KeyT>);
  if (cudaFuncSetAttribute(sort_scatter_kernel<KeyT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(scatter_smem)) != cudaSuccess)
    return B200TBE_ERR_LAUNCH;
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
    sort_histogram_kernel<KeyT><<<tiles, kSortThreads, 0, stream>>>(kin, n, shift, mask, radix,
                                                                   counts, tiles);
    const int st = exclusive_scan_u32(counts, static_cast<int64_t>(radix) * tiles, tile_sums,
                                      nullptr, stream);
    if (st != B200TBE_OK) return st;
    sort_scatter_kernel<KeyT><<<tiles, kSortThreads, scatter_smem, stream>>>(kin, vin, kout, vout, n, shift,
                                                                 mask, radix, bits, counts, tiles);
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
  const int64_t counts = tiles * kMaxRadix;
  return align256(static_cast<size_t>(counts) * 4) +
         align256(static_cast<size_t>(scan_num_tiles(counts)) * 4) + 256;
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
      static_cast<char*>(scratch) + align256(static_cast<size_t>(tiles) * kMaxRadix * 4));
  if (key_bytes == 4)
    return sort_impl<uint32_t>(static_cast<uint32_t*>(keys_a), vals_a,
                               static_cast<uint32_t*>(keys_b), vals_b, n, key_bits, counts,
                               tile_sums, result_in_b, stream);
  return sort_impl<unsigned long long>(static_cast<unsigned long long*>(keys_a), vals_a,
                                       static_cast<unsigned long long*>(keys_b), vals_b, n, key_bits,
                                       counts, tile_sums, result_in_b, stream);
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
constexpr size_t kStaticSortScratchBytes = (size_t{512} * kMaxRadix * 4) + 4096;

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
