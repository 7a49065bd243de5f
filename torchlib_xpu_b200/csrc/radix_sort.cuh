// Internal interface of the hand-written radix sort (radix_sort.cu).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace b200tbe {

// Bytes of scratch sort_pairs needs for n elements.
size_t radix_sort_scratch_bytes(int64_t n);

// Stable LSD radix sort of (key, 32-bit payload) pairs by the low key_bits bits of the key.
// The buffers ping-pong between (keys_a, vals_a) and (keys_b, vals_b), starting in a; *result_in_b
// tells where the sorted data ends up. key_bytes is 4 or 8.
int radix_sort_pairs(void* keys_a, uint32_t* vals_a, void* keys_b, uint32_t* vals_b, int64_t n,
                     int key_bytes, int key_bits, void* scratch, size_t scratch_bytes,
                     bool* result_in_b, cudaStream_t stream);

// ---- segmented form ------------------------------------------------------------------------------
// The array is cut into independent segments and every segment into tiles of kSortPlanTile keys
// (the last tile of a segment may be shorter); all of it is described on the device, so the host
// needs no copy of the segment sizes, only an upper bound on the number of tiles.
constexpr int kSortPlanTile = 4096;   // keys per tile of 4-byte keys

struct SortPlan {
  const uint4* tile_desc;          // [max_tiles] {first key, key count, segment, first tile of the segment}
  const uint32_t* seg_tile_base;   // [segments + 1] exclusive prefix of the tiles per segment
  const uint32_t* total_tiles;     // device scalar: tiles in use (<= max_tiles)
  int max_tiles;                   // the host's bound; sizes the grids
};

size_t radix_sort_planned_scratch_bytes(int64_t max_tiles);

// Upper bound on the tiles of n keys in num_segments segments, and the device memory a plan takes.
int64_t sort_plan_max_tiles(int64_t n, int64_t num_segments);
size_t sort_plan_bytes(int64_t n, int64_t num_segments);

// Builds the plan on the device from segment boundaries offsets[s * stride], s = 0..num_segments
// (int32 or int64, clamped to [0, n]) into plan_mem (sort_plan_bytes, 256-byte aligned). Two small
// kernels, no host read. *seg_start_out receives the device array [num_segments + 1] of boundaries.
// Boundaries that describe more than n keys raise B200TBE_DEV_OFFSETS_NOT_MONOTONE in *status.
int build_sort_plan(const void* offsets, int offset_bytes, int num_segments, int64_t stride, int64_t n,
                    void* plan_mem, int32_t* status, SortPlan* plan, const uint32_t** seg_start_out,
                    cudaStream_t stream);

// Sorts every segment of the plan by the low key_bits bits of its 4-byte keys, stable, keys never
// leaving their segment; passes of at most max_digit_bits (<= 11) bits. Buffers ping-pong as above.
int radix_sort_pairs_planned(uint32_t* keys_a, uint32_t* vals_a, uint32_t* keys_b, uint32_t* vals_b,
                             int64_t n, int key_bits, int max_digit_bits, const SortPlan& plan,
                             void* scratch, size_t scratch_bytes, bool* result_in_b,
                             cudaStream_t stream);

}  // namespace b200tbe
