// Gradient exchange of the table-wise-sharded configuration, as a push: the owner of a gradient
// matrix reads it locally and stores each destination's column block into that peer's matrix through
// its peer mapping (plain 16-byte stores over NVLink, fully coalesced: a row's block is contiguous).
// Stores stream across NVLink while loads are request/response -- pulling the same 0.94 GB measured
// 2.4-2.9 ms on 8 B200s against 1.4 ms for the push -- so only the push is built. No thread waits on
// another GPU: ordering against the destinations' readers is the caller's (stream-ordered barriers).
#include "common.cuh"

namespace b200tbe {
namespace {

struct PushParams {
  const char* src;
  char* dsts[B200TBE_MAX_DESTS];
  int64_t src_stride_bytes;
  int64_t dst_stride_bytes;
  int64_t dst_row_offset;
  int64_t rows;
  int32_t num_dsts;
  int32_t vecs_per_block;   // 16-byte vectors in one destination's column block
};

// Vector i of the source matrix, rows x (num_dsts * vecs_per_block) vectors, goes to destination
// (column block) d at row dst_row_offset + r: consecutive threads read consecutive local vectors
// and write consecutive vectors of one peer row block.
__global__ void __launch_bounds__(256) exchange_push_kernel(const __grid_constant__ PushParams p) {
  const int64_t vecs_per_row = static_cast<int64_t>(p.num_dsts) * p.vecs_per_block;
  const int64_t total = p.rows * vecs_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total;
       i0 += stride * 4) {
    uint4 v[4];
    char* dst[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t i = i0 + u * stride;
      dst[u] = nullptr;
      if (i < total) {
        const int64_t r = i / vecs_per_row;
        const int64_t c = i - r * vecs_per_row;
        const int d = static_cast<int>(c / p.vecs_per_block);
        const int64_t cb = c - static_cast<int64_t>(d) * p.vecs_per_block;
        v[u] = ldg_stream16(p.src + r * p.src_stride_bytes + (c << 4));
        dst[u] = p.dsts[d] + (p.dst_row_offset + r) * p.dst_stride_bytes + (cb << 4);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (dst[u] != nullptr) *reinterpret_cast<uint4*>(dst[u]) = v[u];
  }
}

}  // namespace
}  // namespace b200tbe

using namespace b200tbe;

extern "C" int b200tbe_exchange_push(const b200tbe_exchange_push_params* p,
                                     b200tbe_stream_t stream_) {
  if (p == nullptr || p->src == nullptr) return B200TBE_ERR_BAD_ARG;
  if (p->num_dsts < 1 || p->num_dsts > B200TBE_MAX_DESTS || p->rows < 0 || p->block_bytes < 0 ||
      p->dst_row_offset < 0)
    return B200TBE_ERR_BAD_ARG;
  if (p->rows == 0 || p->block_bytes == 0) return B200TBE_OK;
  if ((p->block_bytes | p->src_stride_bytes | p->dst_stride_bytes) & 15) return B200TBE_ERR_UNSUPPORTED;
  if (p->block_bytes / 16 > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  if (p->src_stride_bytes < p->block_bytes * p->num_dsts || p->dst_stride_bytes < p->block_bytes)
    return B200TBE_ERR_BAD_ARG;
  PushParams d;
  for (int i = 0; i < B200TBE_MAX_DESTS; ++i) {
    d.dsts[i] = i < p->num_dsts ? static_cast<char*>(p->dsts[i]) : nullptr;
    if (i < p->num_dsts && (p->dsts[i] == nullptr || !aligned_to(p->dsts[i], 16)))
      return B200TBE_ERR_BAD_ARG;
  }
  if (!aligned_to(p->src, 16)) return B200TBE_ERR_BAD_ARG;
  d.src = static_cast<const char*>(p->src);
  d.src_stride_bytes = p->src_stride_bytes;
  d.dst_stride_bytes = p->dst_stride_bytes;
  d.dst_row_offset = p->dst_row_offset;
  d.rows = p->rows;
  d.num_dsts = p->num_dsts;
  d.vecs_per_block = static_cast<int32_t>(p->block_bytes / 16);
  exchange_push_kernel<<<kNumSMs * 4, 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(d);
  return launch_status();
}
