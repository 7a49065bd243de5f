// Streaming gather engine shared by the pooled-forward kernels.
//
// A gather of embedding rows is bound by memory latency unless enough bytes are in flight: a
// random 80..512-byte row costs an L2 or HBM round trip of about a microsecond, so an SM needs on
// the order of 100 KB outstanding to keep its share of the memory system busy. Registers cannot
// hold that, shared memory can. Each warp therefore owns a private ring of kStages stages in
// shared memory. To fill a stage, every lane issues ONE bulk asynchronous copy (cp.async.bulk,
// global -> shared, completion counted in bytes on an mbarrier) for the whole row of one lookup,
// so a single warp instruction puts up to 32 rows in flight and costs no registers. The warp
// then consumes stages in order: one row per instruction, lane v taking elements [4v, 4v+4) of the
// row from shared memory, accumulating in fp32 registers, and writing a bag's pooled vector when
// the stream of lookups crosses the bag's end. Two stages are in flight while a third is being
// consumed; 8 warps x 2 stages x 8 KB = 128 KB in flight per SM.
//
// Work is cut into units of a few consecutive bags of one table (so a unit's lookups are one
// contiguous range of the index array and its table parameters are warp-uniform); a persistent
// grid of one CTA per SM strides over the units, which keeps all SMs on the same table at the same
// time and lets repeated rows hit in L2.
//
// Every wait on an mbarrier is bounded: a warp that gives up records B200TBE_DEV_WAIT_TIMEOUT in
// the status word and stops; nothing spins forever.
#pragma once

#include "tbe_pool.cuh"

namespace b200tbe {

constexpr int kStreamWarps = 8;
constexpr int kStreamThreads = kStreamWarps * 32;
constexpr int kStages = 3;
constexpr int kStageBytes = 8192;
constexpr int kWaitSpins = 1 << 22;  // bounded mbarrier wait (each try blocks for a short while)

struct WarpRing {
  alignas(128) char rows[kStages][kStageBytes];
  float weights[kStages][32];
  float2 mult[kStages][32];   // per row {multiplier, bias term} of the stage being consumed
  uint32_t valid[kStages];
  uint32_t pad_;
  unsigned long long bar[kStages];
};

constexpr size_t kStreamSmemBytes = sizeof(WarpRing) * kStreamWarps;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Returns false when the wait gave up.
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, uint32_t parity) {
  for (int i = 0; i < kWaitSpins; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                              unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// Call once per CTA before any warp streams (all threads).
__device__ __forceinline__ void stream_init_rings(WarpRing* rings) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane < kStages) mbar_init(&rings[warp].bar[lane], 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  fence_proxy_async_smem();
  __syncthreads();
}

// What a unit's table looks like to the engine (warp-uniform).
struct StreamTable {
  const char* base;    // row 0
  int64_t stride;      // bytes between rows
  int copy_bytes;      // bytes of a row brought to shared memory (multiple of 16, <= kStageBytes)
  int nvec;            // D / 4: vectors of 4 elements per row
  int64_t num_rows;    // rows in the table, or -1 when indices are not range-checked
};

struct StreamBags {
  const void* indices;
  const void* offsets;
  const float* per_sample_weights;
  int32_t* status;
  int pooling_mode;
};

// ---- shared-memory loads by 32-bit shared address ------------------------------------------------
__device__ __forceinline__ uint32_t lds_u8(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint2 lds_u64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 lds_u128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(a));
  return v;
}
__device__ __forceinline__ float2 lds_f32x2(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
  return v;
}

// ---- row readers ----------------------------------------------------------------------------------
// A reader turns vector v (elements [4v, 4v+4)) of a row in shared memory into two float2 and adds
// them, scaled by sw, to two float2 accumulators. Quantised readers build floats with the
// "magic number" trick: OR-ing a small integer into the mantissa of 2^23 gives 2^23 + q exactly, a
// subtraction gives q -- logic and FMA-pipe instructions only, no int-to-float conversions, and the
// packed f32x2 instructions of sm_100 halve the arithmetic instruction count.
constexpr uint32_t kMagicBits = 0x4B000000u;  // 2^23
constexpr float kMagic = 8388608.f;

struct Acc4 {
  float2 lo, hi;
};

template <typename WT>
struct FloatRow;
template <>
struct FloatRow<float> {
  static constexpr bool kHasHeader = false;
  static constexpr int kHeaderBytes = 0;
  static __device__ __forceinline__ void add(Acc4& a, uint32_t row, int v) {
    const uint4 x = lds_u128(row + (v << 4));
    a.lo = __fadd2_rn(a.lo, make_float2(__uint_as_float(x.x), __uint_as_float(x.y)));
    a.hi = __fadd2_rn(a.hi, make_float2(__uint_as_float(x.z), __uint_as_float(x.w)));
  }
  static __device__ __forceinline__ void fma(Acc4& a, uint32_t row, int v, float sw) {
    const uint4 x = lds_u128(row + (v << 4));
    const float2 s = make_float2(sw, sw);
    a.lo = __ffma2_rn(make_float2(__uint_as_float(x.x), __uint_as_float(x.y)), s, a.lo);
    a.hi = __ffma2_rn(make_float2(__uint_as_float(x.z), __uint_as_float(x.w)), s, a.hi);
  }
};
template <>
struct FloatRow<__half> {
  static constexpr bool kHasHeader = false;
  static constexpr int kHeaderBytes = 0;
  static __device__ __forceinline__ void add(Acc4& a, uint32_t row, int v) {
    const uint2 x = lds_u64(row + (v << 3));
    a.lo = __fadd2_rn(a.lo, half2_bits_to_float2(x.x));
    a.hi = __fadd2_rn(a.hi, half2_bits_to_float2(x.y));
  }
  static __device__ __forceinline__ void fma(Acc4& a, uint32_t row, int v, float sw) {
    const uint2 x = lds_u64(row + (v << 3));
    const float2 s = make_float2(sw, sw);
    a.lo = __ffma2_rn(half2_bits_to_float2(x.x), s, a.lo);
    a.hi = __ffma2_rn(half2_bits_to_float2(x.y), s, a.hi);
  }
};

template <int kBits>
struct QuantRow;
template <>
struct QuantRow<8> {
  static constexpr bool kHasHeader = true;
  static constexpr int kHeaderBytes = 4;
  static __device__ __forceinline__ void fma(Acc4& a, uint32_t row, int v, float sw) {
    const uint32_t w = lds_u32(row + 4 + (v << 2));
    const float2 neg = make_float2(-kMagic, -kMagic), s = make_float2(sw, sw);
    const float2 q01 = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(w, kMagicBits, 0x7440)),
                                              __uint_as_float(__byte_perm(w, kMagicBits, 0x7441))), neg);
    const float2 q23 = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(w, kMagicBits, 0x7442)),
                                              __uint_as_float(__byte_perm(w, kMagicBits, 0x7443))), neg);
    a.lo = __ffma2_rn(q01, s, a.lo);
    a.hi = __ffma2_rn(q23, s, a.hi);
  }
};
template <>
struct QuantRow<4> {
  static constexpr bool kHasHeader = true;
  static constexpr int kHeaderBytes = 4;
  static __device__ __forceinline__ void fma(Acc4& a, uint32_t row, int v, float sw) {
    // nibble k stays at bit 4k inside the mantissa: the float is 2^23 + 16^k * q, and the factor
    // 16^-k (a power of two, exact) goes into the multiplier
    const uint32_t w = lds_u16(row + 4 + (v << 1));
    const float2 neg = make_float2(-kMagic, -kMagic);
    const float2 q01 = __fadd2_rn(make_float2(__uint_as_float((w & 0x000fu) | kMagicBits),
                                              __uint_as_float((w & 0x00f0u) | kMagicBits)), neg);
    const float2 q23 = __fadd2_rn(make_float2(__uint_as_float((w & 0x0f00u) | kMagicBits),
                                              __uint_as_float((w & 0xf000u) | kMagicBits)), neg);
    a.lo = __ffma2_rn(q01, make_float2(sw, sw * 0.0625f), a.lo);
    a.hi = __ffma2_rn(q23, make_float2(sw * (1.f / 256.f), sw * (1.f / 4096.f)), a.hi);
  }
};
template <>
struct QuantRow<2> {
  static constexpr bool kHasHeader = true;
  static constexpr int kHeaderBytes = 4;
  static __device__ __forceinline__ void fma(Acc4& a, uint32_t row, int v, float sw) {
    const uint32_t w = lds_u8(row + 4 + v);
    const float2 neg = make_float2(-kMagic, -kMagic);
    const float2 q01 = __fadd2_rn(make_float2(__uint_as_float((w & 0x03u) | kMagicBits),
                                              __uint_as_float((w & 0x0cu) | kMagicBits)), neg);
    const float2 q23 = __fadd2_rn(make_float2(__uint_as_float((w & 0x30u) | kMagicBits),
                                              __uint_as_float((w & 0xc0u) | kMagicBits)), neg);
    a.lo = __ffma2_rn(q01, make_float2(sw, sw * 0.25f), a.lo);
    a.hi = __ffma2_rn(q23, make_float2(sw * 0.0625f, sw * (1.f / 64.f)), a.hi);
  }
};

// Where a unit's bags are written.
template <typename OT>
struct StreamOut {
  OT* const* outputs;         // destination buffers (kernel parameter space)
  int64_t output_stride;
  int64_t col;                // output_col_offset + D_offsets[t]
  int64_t rows_per_dest;
};

// n consecutive rows, all valid, no bag boundary inside. kScaled: every row has a {multiplier, bias
// term} pair in the stage's side table (quantised rows and/or per-sample weights).
template <typename Row, int kVPL, bool kScaled>
__device__ __forceinline__ void consume_rows(Acc4 (&acc)[kVPL], float& bias_acc, uint32_t row,
                                             uint32_t mult, int copy_bytes, int n, int nvec,
                                             int lane) {
  constexpr int kU = kVPL == 1 ? 4 : (kVPL == 2 ? 2 : 1);
  int i = 0;
  for (; i + kU <= n; i += kU) {
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      float sw = 1.f;
      if (kScaled) {
        const float2 m = lds_f32x2(mult + 8 * u);
        sw = m.x;
        bias_acc += m.y;
      }
#pragma unroll
      for (int k = 0; k < kVPL; ++k) {
        const int v = k * 32 + lane;
        if (kVPL == 1 || v < nvec) {
          if constexpr (kScaled) {
            Row::fma(acc[k], row + u * copy_bytes, v, sw);
          } else {
            Row::add(acc[k], row + u * copy_bytes, v);
          }
        }
      }
    }
    row += kU * copy_bytes;
    mult += kU * 8;
  }
  for (; i < n; ++i) {
    float sw = 1.f;
    if (kScaled) {
      const float2 m = lds_f32x2(mult);
      sw = m.x;
      bias_acc += m.y;
    }
#pragma unroll
    for (int k = 0; k < kVPL; ++k) {
      const int v = k * 32 + lane;
      if (kVPL == 1 || v < nvec) {
        if constexpr (kScaled) {
          Row::fma(acc[k], row, v, sw);
        } else {
          Row::add(acc[k], row, v);
        }
      }
    }
    row += copy_bytes;
    mult += 8;
  }
}

template <typename Row, bool kScaled>
struct AddOrFma {
  template <int kVPL>
  static __device__ __forceinline__ void run(Acc4 (&acc)[kVPL], float& bias_acc, uint32_t row,
                                             uint32_t mult, int copy_bytes, int n, int nvec,
                                             int lane) {
    consume_rows<Row, kVPL, true>(acc, bias_acc, row, mult, copy_bytes, n, nvec, lane);
  }
};
template <typename Row>
struct AddOrFma<Row, false> {
  template <int kVPL>
  static __device__ __forceinline__ void run(Acc4 (&acc)[kVPL], float& bias_acc, uint32_t row,
                                             uint32_t mult, int copy_bytes, int n, int nvec,
                                             int lane) {
    if (mult != 0) {
      consume_rows<Row, kVPL, true>(acc, bias_acc, row, mult, copy_bytes, n, nvec, lane);
    } else {
      consume_rows<Row, kVPL, false>(acc, bias_acc, row, 0, copy_bytes, n, nvec, lane);
    }
  }
};

// Pools the bags [b0, b0 + nb) of table t (nb <= 31): lookups offsets[t*B+b0] .. offsets[t*B+b0+nb).
// `phases` holds one parity bit per ring stage and lives across units. Returns false if a wait
// timed out (the caller must stop using the ring).
template <typename Row, typename OT, typename IndexT, int kVPL>
__device__ __forceinline__ bool stream_unit(const StreamBags& bags, const StreamTable& tab,
                                            const StreamOut<OT>& out, int64_t bag0, int b0, int nb,
                                            WarpRing& ring, uint32_t& phases, int lane) {
  // lane j holds the start of bag j of the unit (j = nb: the unit's end)
  const int64_t my_off = lane <= nb ? load_index<IndexT>(bags.offsets, bag0 + lane) : 0;
  const int64_t p_begin = __shfl_sync(kFullMask, my_off, 0);
  const int64_t p_end = __shfl_sync(kFullMask, my_off, nb);
  const int rows_per_stage = min(32, kStageBytes / tab.copy_bytes);
  const int64_t num_stages = (p_end - p_begin + rows_per_stage - 1) / rows_per_stage;
  const bool weighted = bags.per_sample_weights != nullptr;
  const bool mean = bags.pooling_mode == B200TBE_POOL_MEAN;
  // rows need a per-row multiplier when they carry a header or the lookups carry weights
  const bool scaled = Row::kHasHeader || weighted;

  Acc4 acc[kVPL];
#pragma unroll
  for (int k = 0; k < kVPL; ++k) acc[k].lo = acc[k].hi = make_float2(0.f, 0.f);
  float bias_acc = 0.f;
  int cur_bag = 0;
  int64_t cur_start = p_begin;
  int64_t cur_end = __shfl_sync(kFullMask, my_off, 1);

  auto flush = [&]() {
    const float scale = (mean && cur_end > cur_start) ? 1.f / static_cast<float>(cur_end - cur_start) : 1.f;
    const int b = b0 + cur_bag;
    const int dest = static_cast<int>(b / out.rows_per_dest);
    OT* dst = out.outputs[dest] + (b - dest * out.rows_per_dest) * out.output_stride + out.col;
#pragma unroll
    for (int k = 0; k < kVPL; ++k) {
      const int v = k * 32 + lane;
      if (v < tab.nvec) {
        const float r[4] = {(acc[k].lo.x + bias_acc) * scale, (acc[k].lo.y + bias_acc) * scale,
                            (acc[k].hi.x + bias_acc) * scale, (acc[k].hi.y + bias_acc) * scale};
        store_pooled<OT, 4>(dst + 4 * v, r);
      }
      acc[k].lo = acc[k].hi = make_float2(0.f, 0.f);
    }
    bias_acc = 0.f;
    ++cur_bag;
    cur_start = cur_end;
    cur_end = __shfl_sync(kFullMask, my_off, (cur_bag + 1) & 31);
  };

  // index of the lookup this lane will issue next, fetched one stage ahead
  int64_t next_idx = 0;
  auto prefetch_index = [&](int64_t stage) {
    const int64_t pos = p_begin + stage * rows_per_stage + lane;
    next_idx = (stage < num_stages && lane < rows_per_stage && pos < p_end)
                   ? load_index<IndexT>(bags.indices, pos)
                   : -1;
  };
  auto issue = [&](int64_t stage) {
    const int slot = static_cast<int>(stage % kStages);
    const int64_t pos = p_begin + stage * rows_per_stage + lane;
    const bool in_stage = lane < rows_per_stage && pos < p_end;
    int64_t idx = next_idx;
    prefetch_index(stage + 1);
    bool ok = in_stage;
    if (in_stage && tab.num_rows >= 0 && (idx < 0 || idx >= tab.num_rows)) {
      atomicOr(bags.status, B200TBE_DEV_INDEX_OUT_OF_RANGE);
      ok = false;
    }
    const uint32_t vmask = __ballot_sync(kFullMask, ok);
    if (weighted) ring.weights[slot][lane] = in_stage ? __ldg(bags.per_sample_weights + pos) : 0.f;
#ifdef B200TBE_STREAM_LDGSTS
    if (lane == 0) ring.valid[slot] = vmask;
    const int chunks = tab.copy_bytes >> 4;
    const int total = rows_per_stage * chunks;
    for (int i0 = 0; i0 < total; i0 += 32) {
      const int i = i0 + lane;
      const int row = i / chunks;
      const int chunk = i - row * chunks;
      const int64_t ridx = __shfl_sync(kFullMask, idx, row & 31);
      if (i < total && ((vmask >> row) & 1u)) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(
                         ring.rows[slot] + row * tab.copy_bytes + (chunk << 4))),
                     "l"(tab.base + ridx * tab.stride + (chunk << 4))
                     : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
#else
    if (lane == 0) {
      ring.valid[slot] = vmask;
      mbar_arrive_expect_tx(&ring.bar[slot], __popc(vmask) * static_cast<uint32_t>(tab.copy_bytes));
    }
    if (ok)
      bulk_copy_g2s(ring.rows[slot] + lane * tab.copy_bytes, tab.base + idx * tab.stride,
                    static_cast<uint32_t>(tab.copy_bytes), &ring.bar[slot]);
#endif
  };

  prefetch_index(0);
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < num_stages) {
      issue(s);
    } else {
#ifdef B200TBE_STREAM_LDGSTS
      asm volatile("cp.async.commit_group;" ::: "memory");
#endif
    }
  }
  __syncwarp();

  for (int64_t stage = 0; stage < num_stages; ++stage) {
    if (stage + kStages - 1 < num_stages) {
      // the slot being refilled was read by ordinary loads in the previous iteration
      fence_proxy_async_smem();
      issue(stage + kStages - 1);
    } else {
#ifdef B200TBE_STREAM_LDGSTS
      asm volatile("cp.async.commit_group;" ::: "memory");
#endif
    }
    __syncwarp();
    const int slot = static_cast<int>(stage % kStages);
#ifdef B200TBE_STREAM_LDGSTS
    asm volatile("cp.async.wait_group %0;" ::"n"(kStages - 1) : "memory");
    __syncwarp();
#else
    if (!mbar_wait_bounded(&ring.bar[slot], (phases >> slot) & 1u)) {
      if (lane == 0) atomicOr(bags.status, B200TBE_DEV_WAIT_TIMEOUT);
      return false;
    }
    phases ^= 1u << slot;
#endif
    const uint32_t vmask = ring.valid[slot];
    const int64_t pos0 = p_begin + stage * rows_per_stage;
    const int nr = p_end - pos0 < rows_per_stage ? static_cast<int>(p_end - pos0) : rows_per_stage;
    const uint32_t rows_addr = smem_u32(ring.rows[slot]);
    uint32_t mult_addr = 0;
    if (scaled) {
      // side table: lane i turns row i's header and weight into {multiplier, bias term}
      float sw = weighted ? ring.weights[slot][lane] : 1.f, bw = 0.f;
      if (Row::kHasHeader) {
        const float2 sb = ((vmask >> lane) & 1u)
                              ? half2_bits_to_float2(lds_u32(rows_addr + lane * tab.copy_bytes))
                              : make_float2(0.f, 0.f);
        bw = sb.y * sw;
        sw *= sb.x;
      }
      ring.mult[slot][lane] = make_float2(sw, bw);
      mult_addr = smem_u32(ring.mult[slot]);
      __syncwarp();
    }
    const bool all_valid = vmask == (nr == 32 ? 0xffffffffu : ((1u << nr) - 1u));
    int r = 0;
    while (r < nr) {
      while (pos0 + r == cur_end) flush();
      const int64_t left_in_bag = cur_end - (pos0 + r);
      const int n = left_in_bag < nr - r ? static_cast<int>(left_in_bag) : nr - r;
      if (all_valid) {
        AddOrFma<Row, Row::kHasHeader>::run(acc, bias_acc, rows_addr + r * tab.copy_bytes,
                                            scaled ? mult_addr + r * 8 : 0, tab.copy_bytes, n,
                                            tab.nvec, lane);
      } else {
        // some lookups of this stage were out of range: their rows were never copied
        for (int i = 0; i < n; ++i) {
          if ((vmask >> (r + i)) & 1u)
            AddOrFma<Row, Row::kHasHeader>::run(acc, bias_acc, rows_addr + (r + i) * tab.copy_bytes,
                                                scaled ? mult_addr + (r + i) * 8 : 0,
                                                tab.copy_bytes, 1, tab.nvec, lane);
        }
      }
      r += n;
    }
    __syncwarp();
  }
  while (cur_bag < nb) flush();
  return true;
}

// Any row layout, alignment or width: the bags of a unit one at a time, 128 columns per pass,
// element (col0 + i*32 + lane) in accumulator i, one scalar load per element straight from global
// memory. Correct everywhere, fast nowhere; tables the streaming path cannot take land here.
template <typename OT, typename IndexT>
__device__ __noinline__ void pool_unit_generic(const void* indices, const void* offsets,
                                               const float* per_sample_weights, int32_t* status,
                                               int pooling_mode, int ty, const char* table,
                                               int64_t row_stride, int D, int64_t num_rows,
                                               OT* const* outputs, int64_t output_stride,
                                               int64_t col, int64_t rows_per_dest, int64_t bag0,
                                               int b0, int nb, int lane) {
  const bool weighted = per_sample_weights != nullptr;
  for (int j = 0; j < nb; ++j) {
    const int64_t start = load_index<IndexT>(offsets, bag0 + j);
    const int64_t end = load_index<IndexT>(offsets, bag0 + j + 1);
    const float scale =
        (pooling_mode == B200TBE_POOL_MEAN && end > start) ? 1.f / static_cast<float>(end - start) : 1.f;
    const int b = b0 + j;
    const int dest = static_cast<int>(b / rows_per_dest);
    OT* dst = outputs[dest] + (b - dest * rows_per_dest) * output_stride + col;
    for (int col0 = 0; col0 < D; col0 += 128) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int64_t pos = start; pos < end; ++pos) {
        const int64_t idx = load_index<IndexT>(indices, pos);
        const float w = weighted ? __ldg(per_sample_weights + pos) : 1.f;
        if (num_rows >= 0 && (idx < 0 || idx >= num_rows)) {
          if (lane == 0 && col0 == 0) atomicOr(status, B200TBE_DEV_INDEX_OUT_OF_RANGE);
          continue;
        }
        const unsigned char* row = reinterpret_cast<const unsigned char*>(table) + idx * row_stride;
        float s = 1.f, bsh = 0.f;
        if (ty == B200TBE_INT8 || ty == B200TBE_INT4 || ty == B200TBE_INT2) {
          const unsigned lo = __ldg(reinterpret_cast<const unsigned short*>(row));
          const unsigned hi = __ldg(reinterpret_cast<const unsigned short*>(row) + 1);
          const float2 sb = half2_bits_to_float2(lo | (hi << 16));
          s = sb.x;
          bsh = sb.y;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int e = col0 + i * 32 + lane;
          if (e < D) {
            float val;
            if (ty == B200TBE_INT8) {
              val = fmaf(static_cast<float>(__ldg(row + 4 + e)), s, bsh);
            } else if (ty == B200TBE_INT4) {
              const unsigned byte = __ldg(row + 4 + (e >> 1));
              val = fmaf(static_cast<float>((byte >> ((e & 1) * 4)) & 0xfu), s, bsh);
            } else if (ty == B200TBE_INT2) {
              const unsigned byte = __ldg(row + 4 + (e >> 2));
              val = fmaf(static_cast<float>((byte >> ((e & 3) * 2)) & 0x3u), s, bsh);
            } else if (ty == B200TBE_FP16) {
              val = __half2float(
                  __ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(row) + e)));
            } else {
              val = __ldg(reinterpret_cast<const float*>(row) + e);
            }
            acc[i] = fmaf(val, w, acc[i]);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int e = col0 + i * 32 + lane;
        if (e < D) dst[e] = to_out(acc[i] * scale, static_cast<OT*>(nullptr));
      }
    }
  }
}

// Host side: bags per unit so that there are a few units per warp of the persistent grid.
inline int stream_bags_per_unit(int64_t T, int64_t B) {
  const int64_t warps = static_cast<int64_t>(kNumSMs) * kStreamWarps;
  int64_t bpu = T * B / (4 * warps);
  if (bpu > 31) bpu = 31;
  if (bpu > B) bpu = B;
  if (bpu < 1) bpu = 1;
  return static_cast<int>(bpu);
}

}  // namespace b200tbe
