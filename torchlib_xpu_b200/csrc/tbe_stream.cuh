// Streaming gather engine: the pooled lookup for rows that do not fit a register gather (float rows
// wider than 512 bytes; INT2, float and wide rows of the quantised lookup) and the backward's run
// reduction for rows of more than 512 elements.
//
// A gather of embedding rows is bound by memory latency unless enough bytes are in flight: a
// random 80..4096-byte row costs an L2 or HBM round trip of about a microsecond, so an SM needs on
// the order of 100 KB outstanding to keep its share of the memory system busy. Registers cannot
// hold that for wide rows, shared memory can. Each warp therefore owns a private ring of kStages
// stages in shared memory. A stage is filled with cp.async (16 bytes per lane, 32 consecutive
// chunks per instruction, through L1 so that the hottest rows hit there; the copies cost no
// registers and complete in order per thread, tracked by cp.async groups). The warp then consumes
// stages in order: one row per instruction, lane v taking elements [4v, 4v+4) of the row from shared
// memory, accumulating in fp32 registers, and writing a bag's pooled vector when the stream of
// lookups crosses the bag's end. Two stages are in flight while a third is being consumed;
// 16 warps x 2 stages x 4 KB = 128 KB in flight per SM.
// (One cp.async.bulk per row was measured instead of cp.async: a bulk copy issued by 32 lanes
// executes as 32 separate copies with about 20 instructions of set-up each, slower for rows of a few
// hundred bytes; it is not built.)
//
// Work is cut into units of a few consecutive bags of one table (so a unit's lookups are one
// contiguous range of the index array and its table parameters are warp-uniform); a persistent
// grid of one CTA per SM strides over the units, which keeps all SMs on the same table at the same
// time and lets repeated rows hit in L2. Nothing in the engine waits on another warp.
#pragma once

#include "tbe_pool.cuh"

namespace b200tbe {

constexpr int kStreamWarps = 16;
constexpr int kStreamThreads = kStreamWarps * 32;
constexpr int kStages = 3;
constexpr int kStageBytes = 4096;

struct WarpRing {
  alignas(128) char rows[kStages][kStageBytes];
  float weights[kStages][32];
  float2 mult[kStages][32];   // per row {multiplier, bias term} of the stage being consumed
  uint32_t valid[kStages];
  uint32_t pad_;
};

constexpr size_t kStreamSmemBytes = sizeof(WarpRing) * kStreamWarps;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
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
    // fp32 accumulator += fp16 element in one instruction (mixed-precision add of sm_100)
    const uint2 x = lds_u64(row + (v << 3));
    asm("{.reg .f16 l0, h0, l1, h1;\n"
        "mov.b32 {l0, h0}, %4;\n"
        "mov.b32 {l1, h1}, %5;\n"
        "add.rn.f32.f16 %0, l0, %0;\n"
        "add.rn.f32.f16 %1, h0, %1;\n"
        "add.rn.f32.f16 %2, l1, %2;\n"
        "add.rn.f32.f16 %3, h1, %3;}\n"
        : "+f"(a.lo.x), "+f"(a.lo.y), "+f"(a.hi.x), "+f"(a.hi.y)
        : "r"(x.x), "r"(x.y));
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

// kN consecutive rows starting at shared address `row`, all valid, all of one bag, fully unrolled:
// the loads of all kN rows are independent of each other. kScaled: every row has a {multiplier,
// bias term} pair in the stage's side table (quantised rows and/or per-sample weights).
template <typename Row, int kVPL, bool kScaled, int kN>
__device__ __forceinline__ void consume_fixed(Acc4 (&acc)[kVPL], float& bias_acc, uint32_t row,
                                              uint32_t mult, int copy_bytes, int nvec, int lane) {
#pragma unroll
  for (int u = 0; u < kN; ++u) {
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
}

// Rows with a header are always scaled; float rows only when the lookups carry weights (mult != 0).
template <typename Row, int kVPL, int kN>
__device__ __forceinline__ void consume(Acc4 (&acc)[kVPL], float& bias_acc, uint32_t row,
                                        uint32_t mult, int copy_bytes, int nvec, int lane) {
  if constexpr (Row::kHasHeader) {
    consume_fixed<Row, kVPL, true, kN>(acc, bias_acc, row, mult, copy_bytes, nvec, lane);
  } else {
    if (mult != 0) {
      consume_fixed<Row, kVPL, true, kN>(acc, bias_acc, row, mult, copy_bytes, nvec, lane);
    } else {
      consume_fixed<Row, kVPL, false, kN>(acc, bias_acc, row, 0, copy_bytes, nvec, lane);
    }
  }
}

// Pools the bags [b0, b0 + nb) of table t (nb <= 31): lookups offsets[t*B+b0] .. offsets[t*B+b0+nb).
// Positions inside the unit are 32-bit offsets from the unit's first lookup (a unit is at most 31
// bags long).
template <typename Row, typename OT, typename IndexT, int kVPL>
__device__ __forceinline__ void stream_unit(const StreamBags& bags, const StreamTable& tab,
                                            const StreamOut<OT>& out, int64_t bag0, int b0, int nb,
                                            WarpRing& ring, int lane) {
  // lane j holds the start of bag j of the unit (j = nb: the unit's end), relative to the unit
  const int64_t my_off64 = lane <= nb ? load_index<IndexT>(bags.offsets, bag0 + lane) : 0;
  const int64_t p_begin = __shfl_sync(kFullMask, my_off64, 0);
  const int my_off = lane <= nb ? static_cast<int>(my_off64 - p_begin) : 0x7fffffff;
  const int total = __shfl_sync(kFullMask, my_off, nb);
  const int rows_per_stage = min(32, kStageBytes / tab.copy_bytes);
  const int num_stages = (total + rows_per_stage - 1) / rows_per_stage;
  const bool weighted = bags.per_sample_weights != nullptr;
  const bool mean = bags.pooling_mode == B200TBE_POOL_MEAN;
  // rows need a per-row multiplier when they carry a header or the lookups carry weights
  const bool scaled = Row::kHasHeader || weighted;
  const IndexT* idx_base = reinterpret_cast<const IndexT*>(bags.indices) + p_begin;
  const float* psw_base = weighted ? bags.per_sample_weights + p_begin : nullptr;

  // destination of the unit's first bag; bags of a unit are consecutive rows of one destination
  // unless the unit straddles a destination boundary
  const int rpd = static_cast<int>(out.rows_per_dest);
  const int dest0 = b0 / rpd;
  const bool one_dest = (b0 + nb - 1) / rpd == dest0;
  OT* dst_next = out.outputs[dest0] + static_cast<int64_t>(b0 - dest0 * rpd) * out.output_stride +
                 out.col + 4 * lane;

  Acc4 acc[kVPL];
#pragma unroll
  for (int k = 0; k < kVPL; ++k) acc[k].lo = acc[k].hi = make_float2(0.f, 0.f);
  float bias_acc = 0.f;
  int cur_bag = 0;
  int cur_start = 0;
  int cur_end = __shfl_sync(kFullMask, my_off, 1);

  auto flush = [&]() {
    const float scale = (mean && cur_end > cur_start) ? 1.f / static_cast<float>(cur_end - cur_start) : 1.f;
    OT* dst = dst_next;
    if (!one_dest) {
      const int b = b0 + cur_bag;
      const int dest = b / rpd;
      dst = out.outputs[dest] + static_cast<int64_t>(b - dest * rpd) * out.output_stride + out.col +
            4 * lane;
    }
#pragma unroll
    for (int k = 0; k < kVPL; ++k) {
      if (k * 32 + lane < tab.nvec) {
        const float r[4] = {(acc[k].lo.x + bias_acc) * scale, (acc[k].lo.y + bias_acc) * scale,
                            (acc[k].hi.x + bias_acc) * scale, (acc[k].hi.y + bias_acc) * scale};
        store_pooled<OT, 4>(dst + 128 * k, r);
      }
      acc[k].lo = acc[k].hi = make_float2(0.f, 0.f);
    }
    bias_acc = 0.f;
    dst_next += out.output_stride;
    ++cur_bag;
    cur_start = cur_end;
    cur_end = __shfl_sync(kFullMask, my_off, (cur_bag + 1) & 31);
  };

  // indices of the lookups this lane will issue in the next kIdxAhead stages: the index loads run
  // that many stages ahead of the row copies, which run kStages - 1 stages ahead of consumption
  constexpr int kIdxAhead = 3;
  int64_t idx_q[kIdxAhead] = {};
  const int chunks = tab.copy_bytes >> 4;                       // 16-byte chunks per row
  const int copy_iters = (rows_per_stage * chunks + 31) >> 5;    // warp instructions per stage
  const int chunk_shift = (chunks & (chunks - 1)) == 0 && chunks <= 32 ? __ffs(chunks) - 1 : -1;
  const int lane_row0 = lane / chunks, lane_chunk0 = lane - lane_row0 * chunks;
  const int row_step = 32 / chunks, chunk_step = 32 - row_step * chunks;
  int issue_pos = lane;   // position (relative) this lane issues in the next stage to be issued
  int issue_slot = 0;
  auto load_idx = [&](int pos) -> int64_t {
    return (lane < rows_per_stage && pos < total) ? static_cast<int64_t>(__ldg(idx_base + pos)) : -1;
  };
  auto issue = [&]() {
    const int slot = issue_slot;
    const int pos = issue_pos;
    const bool in_stage = lane < rows_per_stage && pos < total;
    const int64_t idx = idx_q[0];
#pragma unroll
    for (int q = 0; q + 1 < kIdxAhead; ++q) idx_q[q] = idx_q[q + 1];
    idx_q[kIdxAhead - 1] = load_idx(pos + kIdxAhead * rows_per_stage);
    issue_pos += rows_per_stage;
    issue_slot = issue_slot + 1 == kStages ? 0 : issue_slot + 1;
    bool ok = in_stage;
    if (in_stage && tab.num_rows >= 0 && (idx < 0 || idx >= tab.num_rows)) {
      atomicOr(bags.status, B200TBE_DEV_INDEX_OUT_OF_RANGE);
      ok = false;
    }
    const uint32_t vmask = __ballot_sync(kFullMask, ok);
    if (weighted) ring.weights[slot][lane] = in_stage ? __ldg(psw_base + pos) : 0.f;
    if (lane == 0) ring.valid[slot] = vmask;
    // lane i knows where row i of the stage lives (as a 16-byte chunk number inside the table);
    // the copy itself runs over the stage buffer in 16-byte chunks, 32 consecutive chunks per
    // instruction (coalesced on both sides)
    const int64_t byte_off = idx * tab.stride;
    const uint32_t my_chunk = ok ? static_cast<uint32_t>(byte_off >> 4) : 0xffffffffu;
    const bool wide = __any_sync(kFullMask, ok && (byte_off >> 36) != 0);  // table beyond 64 GB
    uint32_t dst = smem_u32(ring.rows[slot]) + (lane << 4);
    if (wide) {
      const char* my_src = ok ? tab.base + byte_off : nullptr;
      int row = lane_row0, chunk = lane_chunk0;
      for (int it = 0; it < copy_iters; ++it) {
        const char* src = reinterpret_cast<const char*>(
            __shfl_sync(kFullMask, reinterpret_cast<unsigned long long>(my_src), row & 31));
        if (row < rows_per_stage && src != nullptr)
          asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src + (chunk << 4))
                       : "memory");
        row += row_step;
        chunk += chunk_step;
        if (chunk >= chunks) {
          chunk -= chunks;
          ++row;
        }
        dst += 512;
      }
    } else if (chunk_shift >= 1) {
      // chunks per row is a power of two (at least 2): a lane copies a pair of adjacent chunks, so
      // one shuffle and one address serve 32 bytes; 64 / chunks rows move per instruction pair
      const int pair_shift = chunk_shift - 1;
      const int rows_per_it = 32 >> pair_shift;
      const char* lane_base = tab.base + ((lane & ((1 << pair_shift) - 1)) << 5);
      uint32_t dst2 = smem_u32(ring.rows[slot]) + (lane << 5);
      const int iters2 = (copy_iters + 1) >> 1;
      int row = lane >> pair_shift;
      for (int it = 0; it < iters2; ++it) {
        const uint32_t c = __shfl_sync(kFullMask, my_chunk, row & 31);
        if (row < rows_per_stage && c != 0xffffffffu) {
          const char* src = lane_base + (static_cast<uint64_t>(c) << 4);
          asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst2), "l"(src) : "memory");
          asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst2 + 16), "l"(src + 16)
                       : "memory");
        }
        row += rows_per_it;
        dst2 += 1024;
      }
    } else if (chunk_shift == 0) {
      // 16-byte rows: one chunk per lane
      const uint32_t c = my_chunk;
      if (c != 0xffffffffu)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst),
                     "l"(tab.base + (static_cast<uint64_t>(c) << 4))
                     : "memory");
    } else {
      int row = lane_row0, chunk = lane_chunk0;
      for (int it = 0; it < copy_iters; ++it) {
        const uint32_t c = __shfl_sync(kFullMask, my_chunk, row & 31);
        if (row < rows_per_stage && c != 0xffffffffu)
          asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst),
                       "l"(tab.base + ((static_cast<uint64_t>(c) + chunk) << 4))
                       : "memory");
        row += row_step;
        chunk += chunk_step;
        if (chunk >= chunks) {
          chunk -= chunks;
          ++row;
        }
        dst += 512;
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

#pragma unroll
  for (int q = 0; q < kIdxAhead; ++q) idx_q[q] = load_idx(lane + q * rows_per_stage);
  int issued = 0;
  for (; issued < kStages - 1; ++issued) {
    if (issued < num_stages) {
      issue();
    } else {
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
  }
  __syncwarp();

  int slot = 0;
  int pos0 = 0;
  for (int stage = 0; stage < num_stages; ++stage) {
    if (stage + kStages - 1 < num_stages) {
      issue();
    } else {
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    __syncwarp();
    asm volatile("cp.async.wait_group %0;" ::"n"(kStages - 1) : "memory");
    __syncwarp();
    const uint32_t vmask = ring.valid[slot];
    const int nr = total - pos0 < rows_per_stage ? total - pos0 : rows_per_stage;
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
    // groups of kG rows take the unrolled path when no bag ends inside the group; a group that
    // holds a bag boundary (or an invalid row) goes row by row
    constexpr int kG = kVPL == 1 ? 4 : (kVPL == 2 ? 2 : 1);
    int r = 0;
    uint32_t row_addr = rows_addr;
    uint32_t m_addr = mult_addr;
    const int m_step = scaled ? 8 : 0;
    while (r < nr) {
      const int left_in_bag = cur_end - (pos0 + r);
      if (all_valid && left_in_bag >= kG && nr - r >= kG) {
        consume<Row, kVPL, kG>(acc, bias_acc, row_addr, m_addr, tab.copy_bytes, tab.nvec, lane);
        r += kG;
        row_addr += kG * tab.copy_bytes;
        m_addr += kG * m_step;
      } else {
        while (pos0 + r == cur_end) flush();
        // a lookup that was out of range never had its row copied
        if ((vmask >> r) & 1u)
          consume<Row, kVPL, 1>(acc, bias_acc, row_addr, m_addr, tab.copy_bytes, tab.nvec, lane);
        ++r;
        row_addr += tab.copy_bytes;
        m_addr += m_step;
      }
    }
    __syncwarp();
    pos0 += rows_per_stage;
    slot = slot + 1 == kStages ? 0 : slot + 1;
  }
  while (cur_bag < nb) flush();
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
