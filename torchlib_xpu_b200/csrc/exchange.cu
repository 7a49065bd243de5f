// Gradient exchange of the table-wise-sharded configuration: every rank pulls, from each peer's
// gradient matrix [rows_per_src, src_stride], the column block that belongs to its own tables into
// a local [num_srcs * rows_per_src, row_elems] matrix. The peers' matrices are peer-mapped device
// memory (NVLink); the kernel reads them with plain 16-byte loads, fully coalesced (a row's block
// is contiguous), and writes local memory. No thread waits on another GPU: ordering against the
// producers and against the next overwrite is the caller's (stream-ordered barriers).
#include "common.cuh"

namespace b200tbe {
namespace {

struct PullParams {
  const char* srcs[B200TBE_MAX_DESTS];
  char* dst;
  int64_t src_stride_bytes;
  int64_t src_col_offset_bytes;
  int64_t dst_stride_bytes;
  int64_t rows_per_src;
  int32_t num_srcs;
  int32_t vecs_per_row;   // 16-byte vectors in a row block
};

__global__ void __launch_bounds__(256) exchange_pull_kernel(const __grid_constant__ PullParams p) {
  const int64_t total = static_cast<int64_t>(p.num_srcs) * p.rows_per_src * p.vecs_per_row;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total;
       i0 += stride * 4) {
    uint4 v[4];
    int64_t dst_off[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t i = i0 + u * stride;
      dst_off[u] = -1;
      if (i < total) {
        const int64_t row = i / p.vecs_per_row;
        const int c = static_cast<int>(i - row * p.vecs_per_row);
        const int s = static_cast<int>(row / p.rows_per_src);
        const int64_t r = row - s * p.rows_per_src;
        v[u] = ldg_stream16(p.srcs[s] + r * p.src_stride_bytes + p.src_col_offset_bytes +
                            (static_cast<int64_t>(c) << 4));
        dst_off[u] = row * p.dst_stride_bytes + (static_cast<int64_t>(c) << 4);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (dst_off[u] >= 0) *reinterpret_cast<uint4*>(p.dst + dst_off[u]) = v[u];
  }
}

}  // namespace
}  // namespace b200tbe

using namespace b200tbe;

extern "C" int b200tbe_exchange_pull(const b200tbe_exchange_pull_params* p,
                                     b200tbe_stream_t stream_) {
  if (p == nullptr || p->dst == nullptr) return B200TBE_ERR_BAD_ARG;
  if (p->num_srcs < 1 || p->num_srcs > B200TBE_MAX_DESTS || p->rows_per_src < 0 ||
      p->row_bytes < 0)
    return B200TBE_ERR_BAD_ARG;
  if (p->rows_per_src == 0 || p->row_bytes == 0) return B200TBE_OK;
  if ((p->row_bytes | p->src_stride_bytes | p->src_col_offset_bytes | p->dst_stride_bytes) & 15)
    return B200TBE_ERR_UNSUPPORTED;
  if (p->row_bytes / 16 > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  PullParams d;
  for (int i = 0; i < B200TBE_MAX_DESTS; ++i) {
    d.srcs[i] = i < p->num_srcs ? static_cast<const char*>(p->srcs[i]) : nullptr;
    if (i < p->num_srcs && (p->srcs[i] == nullptr || !aligned_to(p->srcs[i], 16)))
      return B200TBE_ERR_BAD_ARG;
  }
  if (!aligned_to(p->dst, 16)) return B200TBE_ERR_BAD_ARG;
  d.dst = static_cast<char*>(p->dst);
  d.src_stride_bytes = p->src_stride_bytes;
  d.src_col_offset_bytes = p->src_col_offset_bytes;
  d.dst_stride_bytes = p->dst_stride_bytes;
  d.rows_per_src = p->rows_per_src;
  d.num_srcs = p->num_srcs;
  d.vecs_per_row = static_cast<int32_t>(p->row_bytes / 16);
  exchange_pull_kernel<<<kNumSMs * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(d);
  return launch_status();
}
