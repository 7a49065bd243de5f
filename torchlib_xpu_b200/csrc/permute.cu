// Segment permutation of jagged data: output segment j is input segment perm[j], copied whole.
// This is the data movement of the input distribution of a table-wise sharded lookup (ids arrive
// grouped by source rank and have to be regrouped by table) and of FBGEMM's permute_2D_sparse_data.
//
// Segments range from empty bags to whole tables, so the work is split by output ELEMENT, not by
// segment: a CTA owns a tile of consecutive output elements, finds the segment of its first element
// by a CTA-wide 256-ary search over the output offsets, walks the segment boundaries of the tile into shared
// memory once, marks which of them holds each element of the tile (first elements marked, a running
// maximum spreads the marks), and then every thread copies elements whose source position is the input
// start of their segment plus their distance from its output start. Reads and writes are coalesced inside
// a segment; per element the traffic is its bytes in and out plus one shared-memory lookup.
#include "common.cuh"

namespace b200tbe {
namespace {

constexpr int kPermThreads = 256;
constexpr int kPermItems = 16;                       // elements per thread
constexpr int kPermTile = kPermThreads * kPermItems;
constexpr int kPermMaxSegs = 2048;                  // segment boundaries a tile keeps in shared memory

template <typename OffT>
__device__ __forceinline__ int64_t load_off(const void* p, int64_t i) {
  return static_cast<int64_t>(reinterpret_cast<const OffT*>(p)[i]);
}

// Largest s in [0, n) with off[s] <= x (off is non-decreasing, off[0] <= x).
template <typename OffT>
__device__ __forceinline__ int64_t segment_of(const void* off, int64_t n, int64_t x) {
  int64_t lo = 0, hi = n - 1;
  while (lo < hi) {
    const int64_t mid = (lo + hi + 1) >> 1;
    if (load_off<OffT>(off, mid) <= x) {
      lo = mid;
    } else {
      hi = mid - 1;
    }
  }
  return lo;
}

template <typename ElemT, typename OffT, typename PermT>
__global__ void __launch_bounds__(kPermThreads)
    permute_segments_kernel(const ElemT* __restrict__ in, ElemT* __restrict__ out,
                            const void* __restrict__ in_offsets, const void* __restrict__ out_offsets,
                            const PermT* __restrict__ perm, int64_t num_segments, int64_t total) {
  __shared__ int64_t seg_out_start[kPermMaxSegs];   // output start of the tile's k-th segment
  __shared__ int64_t seg_in_start[kPermMaxSegs];    // input start of the same segment
  __shared__ int seg_count;
  __shared__ int64_t first_seg;
  const int64_t tile0 = static_cast<int64_t>(blockIdx.x) * kPermTile;
  const int64_t tile1 = tile0 + kPermTile < total ? tile0 + kPermTile : total;
  {
    // the segment of the tile's first element, searched by the whole CTA: 256 probes per round
    // narrow the range 256-fold, so 22 bits of segments take 3 dependent loads instead of 22
    int64_t lo = 0, n = num_segments;
    while (n > 1) {
      const int64_t step = (n + kPermThreads - 1) / kPermThreads;
      const int64_t probe = (static_cast<int64_t>(threadIdx.x) + 1) * step;
      const bool le = probe < n && load_off<OffT>(out_offsets, lo + probe) <= tile0;
      const int64_t c = __syncthreads_count(le);   // the offsets are sorted: the true probes are the first c
      lo += c * step;
      n = n - c * step < step ? n - c * step : step;
    }
    if (threadIdx.x == 0) first_seg = lo;
  }
  __syncthreads();
  // the non-empty segments that intersect the tile, in order; threads take candidates round-robin
  // and a segment's slot is its rank among the non-empty ones, found with a block-wide count
  int64_t s = first_seg;
  int filled = 0;
  bool overflow = false;
  while (true) {
    const int64_t cand = s + threadIdx.x;
    bool live = false;
    int64_t o0 = 0;
    if (cand < num_segments) {
      o0 = load_off<OffT>(out_offsets, cand);
      const int64_t o1 = load_off<OffT>(out_offsets, cand + 1);
      live = o0 < tile1 && o1 > o0 && o1 > tile0;
    }
    // rank of this thread's segment among the live ones of this round
    const unsigned ballot = __ballot_sync(kFullMask, live);
    __shared__ int warp_live[kPermThreads / 32];
    if ((threadIdx.x & 31) == 0) warp_live[threadIdx.x >> 5] = __popc(ballot);
    __syncthreads();
    int before = 0, round_total = 0;
    for (int w = 0; w < kPermThreads / 32; ++w) {
      if (w < static_cast<int>(threadIdx.x >> 5)) before += warp_live[w];
      round_total += warp_live[w];
    }
    const int slot = filled + before + __popc(ballot & ((1u << (threadIdx.x & 31)) - 1u));
    if (live) {
      if (slot < kPermMaxSegs) {
        seg_out_start[slot] = o0;
        seg_in_start[slot] = load_off<OffT>(in_offsets, static_cast<int64_t>(perm[cand]));
      }
    }
    filled += round_total;
    // done when the round reached the end of the segments or a segment that starts past the tile
    const bool last_round = s + kPermThreads >= num_segments ||
                            load_off<OffT>(out_offsets, s + kPermThreads) >= tile1;
    __syncthreads();
    if (filled > kPermMaxSegs) overflow = true;
    if (last_round || overflow) break;
    s += kPermThreads;
  }
  if (threadIdx.x == 0) seg_count = filled < kPermMaxSegs ? filled : kPermMaxSegs;
  __syncthreads();
  const int count = seg_count;
  // Which listed segment holds each element of the tile: every segment marks its first element with
  // its slot (slots grow with the position), and a running maximum over the tile spreads the marks.
  // Thread t scans elements [16 t, 16 t + 16); the carry across threads is a warp / CTA max-scan.
  __shared__ __align__(16) uint16_t slot_of[kPermTile];
  __shared__ int warp_carry[kPermThreads / 32];
  if (!overflow) {
    uint4* z = reinterpret_cast<uint4*>(slot_of);
    for (int q = threadIdx.x; q < kPermTile / 8; q += kPermThreads) z[q] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    for (int k = threadIdx.x; k < count; k += kPermThreads) {
      const int64_t at = seg_out_start[k] - tile0;
      slot_of[at > 0 ? at : 0] = static_cast<uint16_t>(k);
    }
    __syncthreads();
    uint16_t* mine = slot_of + threadIdx.x * kPermItems;
    int run = 0;
#pragma unroll
    for (int j = 0; j < kPermItems; ++j) run = max(run, static_cast<int>(mine[j]));
    int incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(kFullMask, incl, o);
      if ((threadIdx.x & 31) >= o) incl = max(incl, up);
    }
    if ((threadIdx.x & 31) == 31) warp_carry[threadIdx.x >> 5] = incl;
    __syncthreads();
    int carry = __shfl_up_sync(kFullMask, incl, 1);
    if ((threadIdx.x & 31) == 0) carry = 0;
    for (int w = 0; w < static_cast<int>(threadIdx.x >> 5); ++w) carry = max(carry, warp_carry[w]);
#pragma unroll
    for (int j = 0; j < kPermItems; ++j) {
      carry = max(carry, static_cast<int>(mine[j]));
      mine[j] = static_cast<uint16_t>(carry);
    }
    __syncthreads();
  }
  // eight elements at a time: their source positions first, then all eight loads, then the stores
  constexpr int kBatch = 8;
#pragma unroll
  for (int k0 = 0; k0 < kPermItems; k0 += kBatch) {
    int64_t src[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int e = (k0 + u) * kPermThreads + threadIdx.x;
      const int64_t i = tile0 + e;
      src[u] = -1;
      if (i >= tile1) continue;
      if (!overflow) {
        const int slot = slot_of[e];
        src[u] = seg_in_start[slot] + (i - seg_out_start[slot]);
      } else {
        // more segment boundaries in one tile than the table holds (thousands of one-element
        // segments): every element searches the global offsets itself
        // (the last segment that starts at or before i is the non-empty one that holds it)
        const int64_t seg = segment_of<OffT>(out_offsets, num_segments, i);
        src[u] = load_off<OffT>(in_offsets, static_cast<int64_t>(perm[seg])) + (i - load_off<OffT>(out_offsets, seg));
      }
    }
    ElemT v[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u)
      if (src[u] >= 0) v[u] = in[src[u]];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int64_t i = tile0 + static_cast<int64_t>(k0 + u) * kPermThreads + threadIdx.x;
      if (src[u] >= 0) out[i] = v[u];
    }
  }
}

template <typename ElemT, typename OffT>
int launch_perm(const void* in, void* out, const void* in_offsets, const void* out_offsets,
                const void* perm, int perm_bytes, int64_t num_segments, int64_t total,
                cudaStream_t stream) {
  const int64_t ctas = (total + kPermTile - 1) / kPermTile;
  if (ctas > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  if (perm_bytes == 4) {
    permute_segments_kernel<ElemT, OffT, int32_t><<<static_cast<unsigned>(ctas), kPermThreads, 0, stream>>>(
        static_cast<const ElemT*>(in), static_cast<ElemT*>(out), in_offsets, out_offsets,
        static_cast<const int32_t*>(perm), num_segments, total);
  } else {
    permute_segments_kernel<ElemT, OffT, int64_t><<<static_cast<unsigned>(ctas), kPermThreads, 0, stream>>>(
        static_cast<const ElemT*>(in), static_cast<ElemT*>(out), in_offsets, out_offsets,
        static_cast<const int64_t*>(perm), num_segments, total);
  }
  return launch_status();
}

}  // namespace
}  // namespace b200tbe

using namespace b200tbe;

extern "C" int b200tbe_permute_segments(const void* in, void* out, const void* in_offsets,
                                        const void* out_offsets, const void* perm,
                                        int64_t num_segments, int64_t total_elems, int32_t elem_bytes,
                                        int32_t offset_bytes, int32_t perm_bytes,
                                        b200tbe_stream_t stream_) {
  if (num_segments < 0 || total_elems < 0) return B200TBE_ERR_BAD_ARG;
  if (num_segments == 0 || total_elems == 0) return B200TBE_OK;
  if (in == nullptr || out == nullptr || in_offsets == nullptr || out_offsets == nullptr || perm == nullptr)
    return B200TBE_ERR_BAD_ARG;
  if ((offset_bytes != 4 && offset_bytes != 8) || (perm_bytes != 4 && perm_bytes != 8))
    return B200TBE_ERR_BAD_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const bool o64 = offset_bytes == 8;
  switch (elem_bytes) {
    case 8:
      return o64 ? launch_perm<uint64_t, int64_t>(in, out, in_offsets, out_offsets, perm, perm_bytes, num_segments, total_elems, stream)
                 : launch_perm<uint64_t, int32_t>(in, out, in_offsets, out_offsets, perm, perm_bytes, num_segments, total_elems, stream);
    case 4:
      return o64 ? launch_perm<uint32_t, int64_t>(in, out, in_offsets, out_offsets, perm, perm_bytes, num_segments, total_elems, stream)
                 : launch_perm<uint32_t, int32_t>(in, out, in_offsets, out_offsets, perm, perm_bytes, num_segments, total_elems, stream);
    case 2:
      return o64 ? launch_perm<uint16_t, int64_t>(in, out, in_offsets, out_offsets, perm, perm_bytes, num_segments, total_elems, stream)
                 : launch_perm<uint16_t, int32_t>(in, out, in_offsets, out_offsets, perm, perm_bytes, num_segments, total_elems, stream);
    default:
      return B200TBE_ERR_UNSUPPORTED;
  }
}
