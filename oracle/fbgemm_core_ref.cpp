// Harness around the FBGEMM-core CPU kernels that ship inside torch's libtorch_cpu.so -- TEST
// INFRASTRUCTURE, not product code. It exists to (1) pin oracle/tbe_oracle.c against an independent
// implementation of the same arithmetic and (2) serve as the timed CPU arm of bench.py.
//
// fbgemm_gpu's own CPU operators are not available in this environment; these are the kernels
// those operators are built on (FBGEMM include/fbgemm/FbgemmEmbedding.h:95-118 and :152-175,
// include/fbgemm/QuantUtils.h:277-308). Work is split over OpenMP threads by (table, block of bags).
#include <fbgemm/FbgemmEmbedding.h>
#include <fbgemm/QuantUtils.h>
#include <omp.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <vector>

namespace fbgemm {
// Exported by libtorch_cpu.so (FBGEMM src/RefImplementations.cc) but declared in no shipped header.
template <typename DataType, typename IndexType, typename OffsetType>
int rowwise_sparse_adagrad_fused_ref(std::int64_t block_size, std::int64_t output_size,
                                     std::int64_t index_size, std::int64_t data_size, DataType* w,
                                     const float* g, float* h, const IndexType* indices,
                                     const OffsetType* offsets_or_lengths, float epsilon, float lr,
                                     bool use_offsets, bool use_stochastic_rounding,
                                     int emu_vector_size, std::int64_t grad_stride);
}  // namespace fbgemm

namespace {

enum { TY_FP32 = 0, TY_FP16 = 1, TY_INT8 = 2, TY_INT4 = 3, TY_INT2 = 4 };
constexpr int kBagsPerTask = 512;

int64_t round_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

int64_t nbit_row_stride(int ty, int D, int row_alignment) {
  int64_t bytes;
  switch (ty) {
    case TY_INT8: bytes = 4 + D; break;
    case TY_INT4: bytes = 4 + (D + 1) / 2; break;
    case TY_INT2: bytes = 4 + (D + 3) / 4; break;
    case TY_FP16: bytes = 2 * int64_t{D}; break;
    default: bytes = 4 * int64_t{D}; break;
  }
  return round_up(bytes, row_alignment);
}

// Runs `kernel` over the bags [b0, b1) of table t with offsets rebased to the block's first lookup.
template <typename InType, typename Kernel>
bool run_block(const Kernel& kernel, const InType* table, int64_t data_size, int64_t t, int B,
               int64_t b0, int64_t b1, const int64_t* indices, const int64_t* offsets,
               const float* psw, float* out, int64_t out_stride, int D_begin) {
  const int64_t bag0 = t * B + b0;
  const int64_t n_bags = b1 - b0;
  const int64_t base = offsets[bag0];
  std::vector<int64_t> local(n_bags + 1);
  for (int64_t i = 0; i <= n_bags; ++i) local[i] = offsets[bag0 + i] - base;
  return kernel(n_bags, local[n_bags], data_size, table, indices + base, local.data(),
                psw ? psw + base : nullptr, out + b0 * out_stride + D_begin);
}

}  // namespace

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API int ref_num_threads() { return omp_get_max_threads(); }

// The OpenMP runtime is shared by the oracle libraries of the process, so this sets the thread count
// of the C restatement too. Launchers such as torchrun export OMP_NUM_THREADS=1; a timed CPU arm
// states its thread count itself instead of inheriting that.
REF_API void ref_set_num_threads(int n) {
  if (n >= 1) omp_set_num_threads(n);
}

// fp32 / fp16 tables; out fp32 [B, out_stride]. rows_per_table bounds the indices (FBGEMM checks).
REF_API int ref_tbe_forward(const void* dev_weights, int weights_ty, const int64_t* weights_offsets,
                            const int32_t* D_offsets, const int64_t* rows_per_table, int T, int B,
                            const int64_t* indices, const int64_t* offsets, const float* psw,
                            int pooling_mode, float* out, int64_t out_stride) {
  if (weights_ty != TY_FP32 && weights_ty != TY_FP16) return -1;
  int failures = 0;
  const int64_t blocks = (B + kBagsPerTask - 1) / kBagsPerTask;
  for (int t = 0; t < T; ++t) {
    const int D = D_offsets[t + 1] - D_offsets[t];
    auto kf = weights_ty == TY_FP32
                  ? fbgemm::GenerateEmbeddingSpMDMWithStrides<float, int64_t, int64_t, float>(
                        D, psw != nullptr, pooling_mode == 1, 16, false, true, out_stride, -1, true)
                  : typename fbgemm::EmbeddingSpMDMKernelSignature<float, int64_t, int64_t, float>::Type();
    auto kh = weights_ty == TY_FP16
                  ? fbgemm::GenerateEmbeddingSpMDMWithStrides<fbgemm::float16, int64_t, int64_t, float>(
                        D, psw != nullptr, pooling_mode == 1, 16, false, true, out_stride, -1, true)
                  : typename fbgemm::EmbeddingSpMDMKernelSignature<fbgemm::float16, int64_t, int64_t, float>::Type();
#pragma omp parallel for schedule(dynamic, 1) reduction(+ : failures)
    for (int64_t blk = 0; blk < blocks; ++blk) {
      const int64_t b0 = blk * kBagsPerTask, b1 = std::min<int64_t>(B, b0 + kBagsPerTask);
      bool ok;
      if (weights_ty == TY_FP32) {
        ok = run_block(kf, static_cast<const float*>(dev_weights) + weights_offsets[t],
                       rows_per_table[t], t, B, b0, b1, indices, offsets, psw, out, out_stride,
                       D_offsets[t]);
      } else {
        ok = run_block(kh, static_cast<const fbgemm::float16*>(dev_weights) + weights_offsets[t],
                       rows_per_table[t], t, B, b0, b1, indices, offsets, psw, out, out_stride,
                       D_offsets[t]);
      }
      failures += ok ? 0 : 1;
    }
  }
  return failures;
}

// Quantised op: INT8 rows go through the 8-bit SpMDM with the header-first fp16 scale/bias
// layout, INT4 / INT2 through the N-bit SpMDM, FP16 / FP32 rows through the float kernels.
REF_API int ref_nbit_forward(const uint8_t* dev_weights, const int64_t* weights_offsets,
                             const uint8_t* weights_tys, const int32_t* D_offsets,
                             const int64_t* rows_per_table, int row_alignment, int T, int B,
                             const int64_t* indices, const int64_t* offsets, const float* psw,
                             int pooling_mode, float* out, int64_t out_stride) {
  int failures = 0;
  const int64_t blocks = (B + kBagsPerTask - 1) / kBagsPerTask;
  const bool hw = psw != nullptr, norm = pooling_mode == 1;
  for (int t = 0; t < T; ++t) {
    const int ty = weights_tys[t];
    const int D = D_offsets[t + 1] - D_offsets[t];
    const int64_t stride = nbit_row_stride(ty, D, row_alignment);
    const uint8_t* table = dev_weights + weights_offsets[t];
    typename fbgemm::EmbeddingSpMDMKernelSignature<uint8_t, int64_t, int64_t, float>::Type kq;
    typename fbgemm::EmbeddingSpMDMKernelSignature<float, int64_t, int64_t, float>::Type kf;
    typename fbgemm::EmbeddingSpMDMKernelSignature<fbgemm::float16, int64_t, int64_t, float>::Type kh;
    if (ty == TY_INT8) {
      kq = fbgemm::GenerateEmbeddingSpMDMWithStrides<uint8_t, int64_t, int64_t, float>(
          D, hw, norm, 16, false, true, out_stride, stride, /*scale_bias_last=*/false);
    } else if (ty == TY_INT4 || ty == TY_INT2) {
      kq = fbgemm::GenerateEmbeddingSpMDMNBitWithStrides<int64_t, int64_t, float>(
          ty == TY_INT4 ? 4 : 2, D, hw, norm, 16, false, true, out_stride, stride,
          /*scale_bias_last=*/false);
    } else if (ty == TY_FP16) {
      kh = fbgemm::GenerateEmbeddingSpMDMWithStrides<fbgemm::float16, int64_t, int64_t, float>(
          D, hw, norm, 16, false, true, out_stride, stride / 2, true);
    } else {
      kf = fbgemm::GenerateEmbeddingSpMDMWithStrides<float, int64_t, int64_t, float>(
          D, hw, norm, 16, false, true, out_stride, stride / 4, true);
    }
#pragma omp parallel for schedule(dynamic, 1) reduction(+ : failures)
    for (int64_t blk = 0; blk < blocks; ++blk) {
      const int64_t b0 = blk * kBagsPerTask, b1 = std::min<int64_t>(B, b0 + kBagsPerTask);
      bool ok;
      if (ty == TY_FP16) {
        ok = run_block(kh, reinterpret_cast<const fbgemm::float16*>(table), rows_per_table[t], t, B,
                       b0, b1, indices, offsets, psw, out, out_stride, D_offsets[t]);
      } else if (ty == TY_FP32) {
        ok = run_block(kf, reinterpret_cast<const float*>(table), rows_per_table[t], t, B, b0, b1,
                       indices, offsets, psw, out, out_stride, D_offsets[t]);
      } else {
        ok = run_block(kq, table, rows_per_table[t], t, B, b0, b1, indices, offsets, psw, out,
                       out_stride, D_offsets[t]);
      }
      failures += ok ? 0 : 1;
    }
  }
  return failures;
}

// Row-wise min-max quantisation by FBGEMM (scale and bias land at the END of its rows) re-packed
// into the header-first TBE layout with the given row alignment.
REF_API int ref_quantize_rows(const float* src, int64_t rows, int D, int ty, int row_alignment,
                              uint8_t* dst) {
  if (ty != TY_INT8 && ty != TY_INT4 && ty != TY_INT2) return -1;
  const int bits = ty == TY_INT8 ? 8 : (ty == TY_INT4 ? 4 : 2);
  const int64_t payload = (int64_t{D} * bits + 7) / 8;
  const int64_t stride = nbit_row_stride(ty, D, row_alignment);
  const int64_t chunk = 4096;
#pragma omp parallel for schedule(static)
  for (int64_t r0 = 0; r0 < rows; r0 += chunk) {
    const int64_t n = std::min(chunk, rows - r0);
    std::vector<uint8_t> tmp((payload + 4) * n);
    fbgemm::FloatOrHalfToFusedNBitRowwiseQuantizedSBHalf<float>(bits, src + r0 * D, n, D,
                                                                 tmp.data());
    for (int64_t r = 0; r < n; ++r) {
      uint8_t* row = dst + (r0 + r) * stride;
      std::memset(row, 0, stride);
      std::memcpy(row, tmp.data() + r * (payload + 4) + payload, 4);
      std::memcpy(row + 4, tmp.data() + r * (payload + 4), payload);
    }
  }
  return 0;
}

// Dequantises header-first rows (row_alignment 1, i.e. stride = 4 + payload) with FBGEMM's
// unoptimised dequantiser (the vectorised one in this torch build mis-reads header-first rows).
REF_API int ref_dequantize_rows(const uint8_t* src, int64_t rows, int D, int ty, float* dst) {
  if (ty != TY_INT8 && ty != TY_INT4 && ty != TY_INT2) return -1;
  const int bits = ty == TY_INT8 ? 8 : (ty == TY_INT4 ? 4 : 2);
  const int64_t payload = (int64_t{D} * bits + 7) / 8;
  fbgemm::FusedNBitRowwiseQuantizedSBHalfToFloatOrHalfRef<float>(
      bits, src, rows, static_cast<int>(payload + 4), dst, /*scale_bias_last=*/false);
  return 0;
}

// FBGEMM's fused row-wise Adagrad reference (per-lookup updates, no de-duplication). Its step is
// w += lr_signed * g / (sqrt(h) + eps): pass lr_signed = -learning_rate for descent.
REF_API int ref_rowwise_adagrad_fused(int weights_ty, int64_t D, int64_t num_bags, int64_t num_indices,
                                      int64_t num_rows, void* w, const float* g, float* h,
                                      const int64_t* indices, const int64_t* offsets, float eps,
                                      float lr_signed, int64_t grad_stride) {
  if (weights_ty == TY_FP32)
    return fbgemm::rowwise_sparse_adagrad_fused_ref<float, int64_t, int64_t>(
        D, num_bags, num_indices, num_rows, static_cast<float*>(w), g, h, indices, offsets, eps,
        lr_signed, true, false, 8, grad_stride);
  if (weights_ty == TY_FP16)
    return fbgemm::rowwise_sparse_adagrad_fused_ref<fbgemm::float16, int64_t, int64_t>(
        D, num_bags, num_indices, num_rows, static_cast<fbgemm::float16*>(w), g, h, indices,
        offsets, eps, lr_signed, true, false, 8, grad_stride);
  return -1;
}
