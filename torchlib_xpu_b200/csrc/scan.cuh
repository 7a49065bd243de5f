// Device-wide exclusive prefix sum over uint32 arrays, as three small kernels (tile sums, scan of
// the tile sums by one CTA, rescan of each tile with its base). No inter-CTA waiting anywhere.
#pragma once

#include "common.cuh"

namespace b200tbe {

constexpr int kScanThreads = 1024;
constexpr int kScanItems = 4;
constexpr int kScanTile = kScanThreads * kScanItems;  // elements per CTA

inline int64_t scan_num_tiles(int64_t n) { return (n + kScanTile - 1) / kScanTile; }

// Exclusive scan of one value per thread across the CTA; returns the prefix of the caller and
// leaves the CTA total in *total (valid for every thread after the call).
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* total) {
  __shared__ uint32_t warp_sums[32];
  __shared__ uint32_t block_total;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t up = __shfl_up_sync(kFullMask, incl, o);
    if (lane >= o) incl += up;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const int nwarps = (blockDim.x + 31) >> 5;
    uint32_t w = lane < nwarps ? warp_sums[lane] : 0;
    uint32_t wincl = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t up = __shfl_up_sync(kFullMask, wincl, o);
      if (lane >= o) wincl += up;
    }
    warp_sums[lane] = wincl - w;
    if (lane == 31) block_total = wincl;
  }
  __syncthreads();
  const uint32_t prefix = warp_sums[warp] + incl - v;
  *total = block_total;
  __syncthreads();  // warp_sums / block_total may be reused by the next call
  return prefix;
}

static __global__ void __launch_bounds__(kScanThreads)
    scan_tile_sums_kernel(const uint32_t* __restrict__ data, int64_t n,
                          uint32_t* __restrict__ tile_sums) {
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile + threadIdx.x * kScanItems;
  uint32_t s = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i)
    if (base + i < n) s += data[base + i];
  uint32_t total;
  block_exclusive_scan(s, &total);
  if (threadIdx.x == 0) tile_sums[blockIdx.x] = total;
}

// In-place exclusive scan of `count` values by a single CTA; the grand total goes to *total_out
// when that is not null.
static __global__ void __launch_bounds__(kScanThreads)
    scan_single_cta_kernel(uint32_t* __restrict__ vals, int64_t count, uint32_t* total_out) {
  uint32_t carry = 0;
  for (int64_t base = 0; base < count; base += kScanThreads) {
    const int64_t i = base + threadIdx.x;
    const uint32_t v = i < count ? vals[i] : 0;
    uint32_t total;
    const uint32_t prefix = block_exclusive_scan(v, &total);
    if (i < count) vals[i] = carry + prefix;
    carry += total;
  }
  if (threadIdx.x == 0 && total_out != nullptr) *total_out = carry;
}

static __global__ void __launch_bounds__(kScanThreads)
    scan_apply_kernel(uint32_t* __restrict__ data, int64_t n,
                      const uint32_t* __restrict__ tile_bases) {
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile + threadIdx.x * kScanItems;
  uint32_t v[kScanItems];
  uint32_t s = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    v[i] = base + i < n ? data[base + i] : 0;
    s += v[i];
  }
  uint32_t total;
  uint32_t prefix = block_exclusive_scan(s, &total) + tile_bases[blockIdx.x];
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    if (base + i < n) data[base + i] = prefix;
    prefix += v[i];
  }
}

// data[0..n) <- exclusive prefix sums, in place. tile_sums needs scan_num_tiles(n) entries.
inline int exclusive_scan_u32(uint32_t* data, int64_t n, uint32_t* tile_sums, uint32_t* total_out,
                              cudaStream_t stream) {
  if (n <= 0) return B200TBE_OK;
  const int64_t tiles = scan_num_tiles(n);
  if (tiles > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  scan_tile_sums_kernel<<<static_cast<unsigned>(tiles), kScanThreads, 0, stream>>>(data, n, tile_sums);
  scan_single_cta_kernel<<<1, kScanThreads, 0, stream>>>(tile_sums, tiles, total_out);
  scan_apply_kernel<<<static_cast<unsigned>(tiles), kScanThreads, 0, stream>>>(data, n, tile_sums);
  return launch_status();
}

}  // namespace b200tbe
