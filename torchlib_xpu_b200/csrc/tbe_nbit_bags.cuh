// Quantised-inference lookup for the common tables: INT8 and INT4 rows of at most 128 elements.
//
// One warp per group of consecutive bags in a plain grid, no shared memory. A row is {fp16 scale, fp16 bias} followed by
// the codes, so the codes start 4 bytes into a 16-byte aligned row: they cannot be fetched with
// aligned 16-byte vectors without dragging the header and the padding through the arithmetic. They
// can be fetched as 32-bit words, which is how this kernel reads them: half a warp takes one row,
// lane w of the half loads code word w (INT8: also word w + 16) and the header word, which all 16
// lanes read from the same address (one broadcast transaction), so EVERY lane dequantises payload:
// 8 elements per lane and row for D = 128 in either type. Two rows (one per half-warp) travel
// through each instruction, several steps' loads are issued before the first is used, and loads
// allocate in L1, where the head of a skewed id stream stays.
//
// Arithmetic per element: the code becomes an exact fp16 integer (byte or nibble dropped into the
// mantissa of 1024.0, then minus 1024 -- for the nibbles that sit 4 bits up, times 1/16 minus 64),
// and one mixed-precision fma adds code x scale, both fp16, into the fp32 sum: the product is
// exact, the sum is rounded once, as in q * scale + bias evaluated in fp32. The biases of a bag's
// rows are summed once per row and added to every element at the end.
//
// Part of tbe_nbit.cu: included there inside its namespace, after NbitParams.
#pragma once

// One warp per CTA, 32 CTAs per SM: a CTA holds its slot until its longest bag is done, so one-warp
// CTAs keep every slot busy, and 64 registers per thread hold eight (INT8) or sixteen (INT4) rows'
// words in flight per warp. Measured on 64 tables: 1.80 ms, against 1.93 ms for two-warp CTAs at
// 48 warps per SM with half as many rows in flight, and 2.05 ms for eight-warp CTAs.
constexpr int kNbitBagWarps = 1;
constexpr int kNbitBagThreads = kNbitBagWarps * 32;
constexpr int kNbitBagCtasPerSm = 32;
constexpr int kNbitBagMaxD = 128;

// Tables this kernel takes; everything else (INT2, float rows, wider or oddly aligned rows) stays
// on the ring engine. Both kernels evaluate this, so every table is pooled exactly once.
__device__ __forceinline__ bool nbit_bag_path(int ty, int D, const char* table, int64_t row_stride) {
  if (D <= 0 || D > kNbitBagMaxD || (row_stride & 3) != 0 || row_stride > 4096 ||
      (reinterpret_cast<uintptr_t>(table) & 3) != 0)
    return false;
  if (ty == B200TBE_INT8) return (D & 3) == 0;
  if (ty == B200TBE_INT4) return (D & 7) == 0;
  return false;
}

__device__ __forceinline__ uint32_t ldg_cached4(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// a[i] += code i * scale for the eight codes held as four half2 {q0: codes 0,1; q1: 2,3; q2: 4,5;
// q3: 6,7} (exact fp16 integers), scale = low half of hdr; bias_sum += bias = high half of hdr. One
// block, so every register pair is split into its halves once.
__device__ __forceinline__ void fma_codes8(float (&a)[8], float& bias_sum, uint32_t q0, uint32_t q1,
                                           uint32_t q2, uint32_t q3, uint32_t hdr) {
  asm("{.reg .f16 s, b, x0, x1, x2, x3, x4, x5, x6, x7;\n"
      "mov.b32 {s, b}, %9;\n"
      "mov.b32 {x0, x1}, %10;\n"
      "mov.b32 {x2, x3}, %11;\n"
      "mov.b32 {x4, x5}, %12;\n"
      "mov.b32 {x6, x7}, %13;\n"
      "fma.rn.f32.f16 %0, x0, s, %0;\n"
      "fma.rn.f32.f16 %1, x1, s, %1;\n"
      "fma.rn.f32.f16 %2, x2, s, %2;\n"
      "fma.rn.f32.f16 %3, x3, s, %3;\n"
      "fma.rn.f32.f16 %4, x4, s, %4;\n"
      "fma.rn.f32.f16 %5, x5, s, %5;\n"
      "fma.rn.f32.f16 %6, x6, s, %6;\n"
      "fma.rn.f32.f16 %7, x7, s, %7;\n"
      "add.rn.f32.f16 %8, b, %8;}\n"
      : "+f"(a[0]), "+f"(a[1]), "+f"(a[2]), "+f"(a[3]), "+f"(a[4]), "+f"(a[5]), "+f"(a[6]), "+f"(a[7]),
        "+f"(bias_sum)
      : "r"(hdr), "r"(q0), "r"(q1), "r"(q2), "r"(q3));
}

__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Four bytes -> two half2 of exact integers: {b0, b1}, {b2, b3}.
__device__ __forceinline__ void bytes_to_half2(uint32_t w, uint32_t& q01, uint32_t& q23) {
  const __half2 k1024 = bits_h2(0x64006400u);
  q01 = h2_bits(__hsub2(bits_h2(__byte_perm(w, 0x64646464u, 0x4140)), k1024));
  q23 = h2_bits(__hsub2(bits_h2(__byte_perm(w, 0x64646464u, 0x4342)), k1024));
}

// Eight nibbles n0..n7 (n0 = lowest 4 bits) -> four half2 of exact integers:
// {n0, n4}, {n1, n5}, {n2, n6}, {n3, n7}.
__device__ __forceinline__ void nibbles_to_half2(uint32_t w, uint32_t (&q)[4]) {
  const __half2 k1024 = bits_h2(0x64006400u);
  const __half2 k16th = bits_h2(0x2c002c00u);   // 1/16
  const __half2 k64 = bits_h2(0x54005400u);     // 64
  const uint32_t hi = w >> 8;
  q[0] = h2_bits(__hsub2(bits_h2((w & 0x000f000fu) | 0x64006400u), k1024));
  q[1] = h2_bits(__hfma2(bits_h2((w & 0x00f000f0u) | 0x64006400u), k16th, __hneg2(k64)));
  q[2] = h2_bits(__hsub2(bits_h2((hi & 0x000f000fu) | 0x64006400u), k1024));
  q[3] = h2_bits(__hfma2(bits_h2((hi & 0x00f000f0u) | 0x64006400u), k16th, __hneg2(k64)));
}

// One row's words into the running sums. INT8: w0 = elements e0..e0+3 -> a[0..3], w1 = the word 64
// elements on -> a[4..7]. INT4: w0 = nibbles n0..n7 -> a[2i] += n_i, a[2i + 1] += n_(i+4) (w1 unused).
template <bool kInt4, bool kWeighted>
__device__ __forceinline__ void add_quantised_row(float (&a)[8], float& bias_sum, uint32_t hdr, uint32_t w0,
                                                  uint32_t w1, float weight) {
  if (kInt4) {
    uint32_t q[4];
    nibbles_to_half2(w0, q);
    if (kWeighted) {
      const float s = __half2float(__ushort_as_half(static_cast<unsigned short>(hdr & 0xffffu))) * weight;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = half2_bits_to_float2(q[i]);
        a[2 * i] = fmaf(f.x, s, a[2 * i]);
        a[2 * i + 1] = fmaf(f.y, s, a[2 * i + 1]);
      }
    } else {
      fma_codes8(a, bias_sum, q[0], q[1], q[2], q[3], hdr);
    }
  } else {
    uint32_t q01, q23, q45, q67;
    bytes_to_half2(w0, q01, q23);
    bytes_to_half2(w1, q45, q67);
    if (kWeighted) {
      const float s = __half2float(__ushort_as_half(static_cast<unsigned short>(hdr & 0xffffu))) * weight;
      const float2 f0 = half2_bits_to_float2(q01), f1 = half2_bits_to_float2(q23),
                   f2 = half2_bits_to_float2(q45), f3 = half2_bits_to_float2(q67);
      a[0] = fmaf(f0.x, s, a[0]);
      a[1] = fmaf(f0.y, s, a[1]);
      a[2] = fmaf(f1.x, s, a[2]);
      a[3] = fmaf(f1.y, s, a[3]);
      a[4] = fmaf(f2.x, s, a[4]);
      a[5] = fmaf(f2.y, s, a[5]);
      a[6] = fmaf(f3.x, s, a[6]);
      a[7] = fmaf(f3.y, s, a[7]);
    } else {
      fma_codes8(a, bias_sum, q01, q23, q45, q67, hdr);
    }
  }
  if (kWeighted)
    bias_sum = fmaf(__half2float(__ushort_as_half(static_cast<unsigned short>(hdr >> 16))), weight, bias_sum);
}

// Pools bags [bag0, bag0 + nb), nb <= 32, of one table (bag0 = t * B + b0) as one stream of lookups,
// as pool_float_bags does for float rows: rounds of 2 * kSteps rows whatever the bags' lengths, the
// next 32 ids requested before the current ones' rows, a bag closed (sum of the two half-warps, plus
// the bias sum, stored) at the step that holds its last lookup.
// kFull: D = 128, every lane of a half-warp has its code words (no lane sits out).
template <typename OT, typename IndexT, bool kInt4, bool kWeighted, bool kFull>
__device__ __forceinline__ void pool_quantised_bags(const NbitParams& p, const char* table, uint32_t row_stride,
                                                    int D, int64_t num_rows, int64_t col, int64_t bag0, int b0,
                                                    int nb, int lane) {
  constexpr int kSteps = kInt4 ? 8 : 4;   // rows per half-warp whose words are in flight
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
  const int half = lane >> 4, w = lane & 15;
  // this lane's code words: INT4 word w = elements 8w..8w+7; INT8 words w and w + 16 = elements
  // 4w..4w+3 and 64+4w..64+4w+3
  const bool on0 = kFull || (kInt4 ? 8 * w < D : 4 * w < D);
  const bool on1 = !kInt4 && (kFull || 64 + 4 * w < D);
  const char* lane_base = table + 4 + 4 * w;
  const int64_t row_limit = num_rows >= 0 ? num_rows : int64_t{0xffffffff};
  const bool mean = p.pooling_mode == B200TBE_POOL_MEAN;
  const int rpd = static_cast<int>(p.rows_per_dest);

  float a[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) a[e] = 0.f;
  float bias_sum = 0.f;
  int cur = 0;                                              // bag being summed (warp-uniform)
  int cur_start = 0;
  int cur_end = __shfl_sync(kFullMask, my_end, 0);

  // where bag `cur` goes: consecutive bags are consecutive rows of a destination
  int dest = b0 / rpd;
  int row_in_dest = b0 - dest * rpd;
  OT* dst = reinterpret_cast<OT* const*>(p.outputs)[dest] + static_cast<int64_t>(row_in_dest) * p.output_stride + col;

  // closes bag `cur`: each half-warp keeps half of its lanes' sums (INT8: half 0 the first code word's
  // elements, half 1 the second's; INT4: the word's low and high four elements), so one exchange of
  // four values and the bias sum does it
  auto close_bag = [&]() {
    const int pooled = cur_end - cur_start;   // MEAN divides by the bag's length, skipped ids included
    const float scale = (mean && pooled > 0) ? 1.f / static_cast<float>(pooled) : 1.f;
    bias_sum += __shfl_xor_sync(kFullMask, bias_sum, 16);
    float r[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      // nibbles_to_half2 pairs nibble i with nibble i + 4: a[2i] = element 8w + i, a[2i + 1] = element 8w + 4 + i
      const int keep0 = kInt4 ? 2 * e : e, keep1 = kInt4 ? 2 * e + 1 : e + 4;
      const float other = __shfl_xor_sync(kFullMask, half ? a[keep0] : a[keep1], 16);
      r[e] = ((half ? a[keep1] : a[keep0]) + other + bias_sum) * scale;
    }
    if (kInt4) {
      if (on0) store_pooled<OT, 4>(dst + 8 * w + 4 * half, r);
    } else {
      if (half ? on1 : on0) store_pooled<OT, 4>(dst + 64 * half + 4 * w, r);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = 0.f;
    bias_sum = 0.f;
    ++cur;
    cur_start = cur_end;
    cur_end = __shfl_sync(kFullMask, my_end, cur & 31);
    dst += p.output_stride;
    if (++row_in_dest == rpd && cur < nb) {
      row_in_dest = 0;
      dst = reinterpret_cast<OT* const*>(p.outputs)[++dest] + col;
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
    // this lane's row id; a skipped lookup (past the stream's end, id out of range) reads row 0 with
    // its header replaced by zero: scale 0 and bias 0 add nothing, and no load needs a test
    uint32_t my_row = 0;
    bool my_ok = false;
    const float my_w = next_w;
    if (lane < n) {
      const int64_t i = static_cast<int64_t>(next_id);
      if (i < 0 || i >= row_limit) {
        if (p.status != nullptr) atomicOr(p.status, B200TBE_DEV_INDEX_OUT_OF_RANGE);
      } else {
        my_row = static_cast<uint32_t>(i);
        my_ok = true;
      }
    }
    if (c + 32 + lane < total) {
      next_id = __ldg(idx + c + 32 + lane);
      if (kWeighted) next_w = __ldg(psw + c + 32 + lane);
    }
    const uint32_t ok_mask = __ballot_sync(kFullMask, my_ok);
    for (int j = 0; j < n; j += 2 * kSteps) {
      uint32_t hdr[kSteps], w0[kSteps], w1[kSteps];
      float wt[kSteps];
#pragma unroll
      for (int u = 0; u < kSteps; ++u) {
        const int rr = (j + 2 * u + half) & 31;
        const uint32_t row = __shfl_sync(kFullMask, my_row, rr);
        wt[u] = 1.f;
        if (kWeighted) wt[u] = __shfl_sync(kFullMask, my_w, rr);
        const char* src = row_address(lane_base, row, row_stride);
        hdr[u] = ldg_cached4(src - 4 - 4 * w);
        w0[u] = 0u;
        w1[u] = 0u;
        if (on0) w0[u] = ldg_cached4(src);
        if (on1) w1[u] = ldg_cached4(src + 64);
        if (((ok_mask >> rr) & 1u) == 0 || j + 2 * u + half >= 32) hdr[u] = 0u;
      }
      if (c + j + 2 * kSteps < cur_end) {         // the whole round inside the open bag, which goes on
#pragma unroll
        for (int u = 0; u < kSteps; ++u)
          add_quantised_row<kInt4, kWeighted>(a, bias_sum, hdr[u], w0[u], w1[u], wt[u]);
        continue;
      }
#pragma unroll
      for (int u = 0; u < kSteps; ++u) {
        const int step = c + j + 2 * u;           // lookups step and step + 1 of the stream
        if (step + 2 < cur_end) {                 // both inside the open bag, which goes on
          add_quantised_row<kInt4, kWeighted>(a, bias_sum, hdr[u], w0[u], w1[u], wt[u]);
        } else if (j + 2 * u < n) {
          // a bag ends in this step: each row goes to the bag that holds it, bags close in order
          const int q = step + half;
          bool pending = true;
          while (cur < nb) {
            if (pending && q < cur_end) {
              add_quantised_row<kInt4, kWeighted>(a, bias_sum, hdr[u], w0[u], w1[u], wt[u]);
              pending = false;
            }
            if (step + 2 < cur_end) break;
            close_bag();
          }
        }
      }
    }
  }
  while (cur < nb) close_bag();   // bags without lookups at the group's end (or a group without any)
}

template <typename OT, typename IndexT, bool kWeighted>
__global__ void __launch_bounds__(kNbitBagThreads, kNbitBagCtasPerSm)
    tbe_nbit_bags_kernel(const __grid_constant__ NbitParams p) {
  const int lane = threadIdx.x;
  const int t = static_cast<int>(blockIdx.x / static_cast<unsigned>(p.groups_per_table));
  const int b0 = static_cast<int>(blockIdx.x - static_cast<unsigned>(t) * p.groups_per_table) * p.bag_group;
  const int nb = p.B - b0 < p.bag_group ? p.B - b0 : p.bag_group;
  const int64_t bag0 = static_cast<int64_t>(t) * p.B + b0;
  const int ty = __ldg(p.weights_tys + t);
  const int D_begin = __ldg(p.D_offsets + t);
  const int D = __ldg(p.D_offsets + t + 1) - D_begin;
  const char* table = reinterpret_cast<const char*>(p.dev_weights) + __ldg(p.weights_offsets + t);
  const int64_t row_stride = nbit_row_stride(ty, D, p.row_alignment);
  if (!nbit_bag_path(ty, D, table, row_stride)) return;   // the ring engine pools this table
  const int64_t num_rows = p.rows_per_table ? __ldg(p.rows_per_table + t) : -1;
  const int64_t col = p.output_col_offset + D_begin;
  const uint32_t stride = static_cast<uint32_t>(row_stride);   // at most 4 + 128 bytes plus padding
  if (ty == B200TBE_INT4) {
    if (D == kNbitBagMaxD) {
      pool_quantised_bags<OT, IndexT, true, kWeighted, true>(p, table, stride, D, num_rows, col, bag0, b0, nb, lane);
    } else {
      pool_quantised_bags<OT, IndexT, true, kWeighted, false>(p, table, stride, D, num_rows, col, bag0, b0, nb, lane);
    }
  } else {
    if (D == kNbitBagMaxD) {
      pool_quantised_bags<OT, IndexT, false, kWeighted, true>(p, table, stride, D, num_rows, col, bag0, b0, nb, lane);
    } else {
      pool_quantised_bags<OT, IndexT, false, kWeighted, false>(p, table, stride, D, num_rows, col, bag0, b0, nb, lane);
    }
  }
}
