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

}  // namespace b200tbe
