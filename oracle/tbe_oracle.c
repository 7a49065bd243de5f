/*
 * CPU oracle for the TBE / jagged hot path -- TEST INFRASTRUCTURE, not product code.
 *
 * Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may load this library; the
 * product (torchlib_xpu_b200) never does.
 *
 * PARITY UNPINNED against fbgemm_gpu: the intel/torchlib-xpu tree holds no TBE or jagged code, no
 * tests and no golden vectors for this path, and fbgemm_gpu itself is not installed. What this
 * restatement follows instead, and is checked against in tests/test_oracle_pins.py:
 *   - pooling semantics: the pseudocode in FBGEMM's include/fbgemm/FbgemmEmbedding.h:26-38
 *     (out = sum over the bag of row * weight, divided by the length when normalising and
 *     length > 0), offsets convention ibid. :58-62; pinned against the FBGEMM-core kernels that
 *     ship inside torch's libtorch_cpu.so (GenerateEmbeddingSpMDMWithStrides, ibid. :95-118);
 *   - quantised rows: fp16 scale and bias at the beginning of each row (ibid. :90-93, :147-150),
 *     value = q * scale + bias, INT4 element 2i in the low nibble of byte i; pinned against
 *     GenerateEmbeddingSpMDMNBitWithStrides (ibid. :152-175) and
 *     FusedNBitRowwiseQuantizedSBHalfToFloatOrHalf (include/fbgemm/QuantUtils.h:293-308);
 *   - row-wise Adagrad: one momentum per row, m += mean(g^2), w -= lr/(sqrt(m)+eps)*g, the update
 *     of FBGEMM's fused row-wise Adagrad (FbgemmEmbedding.h:297-316), pinned against the
 *     rowwise_sparse_adagrad_fused_ref symbol of libtorch_cpu.so on inputs without repeated rows;
 *     "exact" means repeated rows of a batch are summed first and updated once;
 *   - jagged ops: the contract of ATen's _jagged_to_padded_dense_forward /
 *     _padded_dense_to_jagged_forward, pinned against those CPU ops.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

enum { TY_FP32 = 0, TY_FP16 = 1, TY_INT8 = 2, TY_INT4 = 3, TY_INT2 = 4 };
enum { POOL_SUM = 0, POOL_MEAN = 1 };
enum { OPT_SGD = 0, OPT_ROWWISE_ADAGRAD = 1 };

/* ---- IEEE binary16 <-> binary32, round to nearest even ---------------------------------- */
ORACLE_API float oracle_half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else { /* subnormal: normalise */
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while ((man & 0x400u) == 0);
      man &= 0x3ffu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

ORACLE_API uint16_t oracle_float_to_half(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
  const uint32_t absx = x & 0x7fffffffu;
  if (absx >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (absx > 0x7f800000u ? 0x200u : 0));
  if (absx >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* rounds to inf */
  if (absx < 0x33000001u) return sign;                          /* rounds to zero */
  int exp = (int)(absx >> 23) - 127;
  uint32_t man = (absx & 0x7fffffu) | 0x800000u;
  int shift;
  uint32_t half_exp;
  if (exp < -14) { /* subnormal half */
    shift = 13 + (-14 - exp);
    half_exp = 0;
  } else {
    shift = 13;
    half_exp = (uint32_t)(exp + 15);
  }
  uint32_t q = man >> shift;
  const uint32_t rem = man & ((1u << shift) - 1u);
  const uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
  uint32_t out;
  if (half_exp == 0) {
    out = q; /* may carry into exponent 1, which is the right encoding */
  } else {
    out = ((half_exp - 1) << 10) + q; /* q includes the hidden bit; carry propagates */
  }
  return (uint16_t)(sign | out);
}

static int64_t round_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

/* ---- TBE forward, fp32 / fp16 tables ------------------------------------------------------
 * out is fp32 [B, out_stride]; bag (t, b) = id t*B + b writes columns D_offsets[t] .. */
ORACLE_API int oracle_tbe_forward(const void* dev_weights, int weights_ty,
                                  const int64_t* weights_offsets, const int32_t* D_offsets, int T,
                                  int B, const int64_t* indices, const int64_t* offsets,
                                  const float* per_sample_weights, int pooling_mode, float* out,
                                  int64_t out_stride) {
  if (weights_ty != TY_FP32 && weights_ty != TY_FP16) return -1;
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t bag = 0; bag < (int64_t)T * B; ++bag) {
    const int t = (int)(bag / B);
    const int64_t b = bag % B;
    const int D = D_offsets[t + 1] - D_offsets[t];
    float* o = out + b * out_stride + D_offsets[t];
    for (int d = 0; d < D; ++d) o[d] = 0.f;
    const int64_t start = offsets[bag], end = offsets[bag + 1];
    for (int64_t j = start; j < end; ++j) {
      const int64_t row = weights_offsets[t] + indices[j] * D;
      const float w = per_sample_weights ? per_sample_weights[j] : 1.f;
      if (weights_ty == TY_FP32) {
        const float* src = (const float*)dev_weights + row;
        for (int d = 0; d < D; ++d) o[d] += src[d] * w;
      } else {
        const uint16_t* src = (const uint16_t*)dev_weights + row;
        for (int d = 0; d < D; ++d) o[d] += oracle_half_to_float(src[d]) * w;
      }
    }
    if (pooling_mode == POOL_MEAN && end > start) {
      const float inv = 1.f / (float)(end - start);
      for (int d = 0; d < D; ++d) o[d] *= inv;
    }
  }
  return 0;
}

/* Bytes between consecutive rows of a table in the quantised op. */
ORACLE_API int64_t oracle_nbit_row_stride(int ty, int D, int row_alignment) {
  int64_t bytes;
  switch (ty) {
    case TY_INT8: bytes = 4 + D; break;
    case TY_INT4: bytes = 4 + (D + 1) / 2; break;
    case TY_INT2: bytes = 4 + (D + 3) / 4; break;
    case TY_FP16: bytes = 2 * (int64_t)D; break;
    default: bytes = 4 * (int64_t)D; break;
  }
  return round_up(bytes, row_alignment);
}

/* Element d of one row of a table of type ty. */
static float nbit_element(const uint8_t* row, int ty, int d) {
  if (ty == TY_FP32) {
    float f;
    memcpy(&f, row + 4 * (int64_t)d, 4);
    return f;
  }
  if (ty == TY_FP16) {
    uint16_t h;
    memcpy(&h, row + 2 * (int64_t)d, 2);
    return oracle_half_to_float(h);
  }
  uint16_t hs, hb;
  memcpy(&hs, row, 2);
  memcpy(&hb, row + 2, 2);
  const float scale = oracle_half_to_float(hs), bias = oracle_half_to_float(hb);
  unsigned q;
  if (ty == TY_INT8) {
    q = row[4 + d];
  } else if (ty == TY_INT4) {
    q = (row[4 + d / 2] >> ((d & 1) * 4)) & 0xfu;
  } else {
    q = (row[4 + d / 4] >> ((d & 3) * 2)) & 0x3u;
  }
  return (float)q * scale + bias;
}

/* ---- quantised forward; out fp32 [B, out_stride] ------------------------------------------ */
ORACLE_API int oracle_nbit_forward(const uint8_t* dev_weights, const int64_t* weights_offsets,
                                   const uint8_t* weights_tys, const int32_t* D_offsets,
                                   int row_alignment, int T, int B, const int64_t* indices,
                                   const int64_t* offsets, const float* per_sample_weights,
                                   int pooling_mode, float* out, int64_t out_stride) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t bag = 0; bag < (int64_t)T * B; ++bag) {
    const int t = (int)(bag / B);
    const int64_t b = bag % B;
    const int ty = weights_tys[t];
    const int D = D_offsets[t + 1] - D_offsets[t];
    const int64_t stride = oracle_nbit_row_stride(ty, D, row_alignment);
    float* o = out + b * out_stride + D_offsets[t];
    for (int d = 0; d < D; ++d) o[d] = 0.f;
    const int64_t start = offsets[bag], end = offsets[bag + 1];
    for (int64_t j = start; j < end; ++j) {
      const uint8_t* row = dev_weights + weights_offsets[t] + indices[j] * stride;
      const float w = per_sample_weights ? per_sample_weights[j] : 1.f;
      for (int d = 0; d < D; ++d) o[d] += nbit_element(row, ty, d) * w;
    }
    if (pooling_mode == POOL_MEAN && end > start) {
      const float inv = 1.f / (float)(end - start);
      for (int d = 0; d < D; ++d) o[d] *= inv;
    }
  }
  return 0;
}

/* Row-wise min-max quantisation of rows x D floats into the TBE row layout (header first).
 * scale = (max - min) / (2^bits - 1) and bias = min, both rounded to fp16 before use;
 * q = round((x - bias) / scale) clamped. */
ORACLE_API int oracle_quantize_rows(const float* src, int64_t rows, int D, int ty, int row_alignment,
                                    uint8_t* dst) {
  if (ty != TY_INT8 && ty != TY_INT4 && ty != TY_INT2) return -1;
  const int bits = ty == TY_INT8 ? 8 : (ty == TY_INT4 ? 4 : 2);
  const int qmax = (1 << bits) - 1;
  const int64_t stride = oracle_nbit_row_stride(ty, D, row_alignment);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* x = src + r * D;
    uint8_t* row = dst + r * stride;
    memset(row, 0, (size_t)stride);
    float mn = x[0], mx = x[0];
    for (int d = 1; d < D; ++d) {
      if (x[d] < mn) mn = x[d];
      if (x[d] > mx) mx = x[d];
    }
    const uint16_t hb = oracle_float_to_half(mn);
    const float bias = oracle_half_to_float(hb);
    const float range = mx - bias;
    uint16_t hs = oracle_float_to_half(range == 0.f ? 1.f : range / (float)qmax);
    float scale = oracle_half_to_float(hs);
    if (scale == 0.f) { /* range too small for fp16: fall back to 1 */
      hs = oracle_float_to_half(1.f);
      scale = 1.f;
    }
    memcpy(row, &hs, 2);
    memcpy(row + 2, &hb, 2);
    const float inv = 1.f / scale;
    for (int d = 0; d < D; ++d) {
      long q = lrintf((x[d] - bias) * inv);
      if (q < 0) q = 0;
      if (q > qmax) q = qmax;
      if (ty == TY_INT8) {
        row[4 + d] = (uint8_t)q;
      } else if (ty == TY_INT4) {
        row[4 + d / 2] |= (uint8_t)(q << ((d & 1) * 4));
      } else {
        row[4 + d / 4] |= (uint8_t)(q << ((d & 3) * 2));
      }
    }
  }
  return 0;
}

/* ---- stable LSD radix sort of (key, payload) pairs, 16 bits per pass ----------------------- */
static void sort_pairs(uint64_t* keys, uint32_t* vals, int64_t n, int bits) {
  uint64_t* k2 = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)(n > 0 ? n : 1));
  uint32_t* v2 = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)(n > 0 ? n : 1));
  int64_t* count = (int64_t*)malloc(sizeof(int64_t) * 65537);
  uint64_t *ka = keys, *kb = k2;
  uint32_t *va = vals, *vb = v2;
  for (int shift = 0; shift < bits; shift += 16) {
    memset(count, 0, sizeof(int64_t) * 65537);
    for (int64_t i = 0; i < n; ++i) ++count[((ka[i] >> shift) & 0xffffu) + 1];
    for (int i = 0; i < 65536; ++i) count[i + 1] += count[i];
    for (int64_t i = 0; i < n; ++i) {
      const int64_t dst = count[(ka[i] >> shift) & 0xffffu]++;
      kb[dst] = ka[i];
      vb[dst] = va[i];
    }
    uint64_t* tk = ka; ka = kb; kb = tk;
    uint32_t* tv = va; va = vb; vb = tv;
  }
  if (ka != keys) {
    memcpy(keys, ka, sizeof(uint64_t) * (size_t)n);
    memcpy(vals, va, sizeof(uint32_t) * (size_t)n);
  }
  free(k2);
  free(v2);
  free(count);
}

/* ---- TBE backward with the optimizer fused, exact (one update per distinct row) -----------
 * grad is fp32 [B, grad_stride]; weights fp32 or fp16, updated in place; momentum1 fp32. */
ORACLE_API int oracle_tbe_backward(void* dev_weights, int weights_ty, const int64_t* weights_offsets,
                                   const int32_t* D_offsets, const int64_t* hash_size_cumsum, int T,
                                   int B, const int64_t* indices, const int64_t* offsets,
                                   const float* per_sample_weights, int pooling_mode,
                                   const float* grad, int64_t grad_stride, float* momentum1,
                                   const int64_t* momentum1_offsets, int optimizer, float lr,
                                   float eps) {
  if (weights_ty != TY_FP32 && weights_ty != TY_FP16) return -1;
  const int64_t n = offsets[(int64_t)T * B];
  uint64_t* keys = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)(n > 0 ? n : 1));
  uint32_t* pos = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)(n > 0 ? n : 1));
  int32_t* bag_of = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n > 0 ? n : 1));
  if (n > 0xffffffffLL) return -2;
  for (int64_t bag = 0; bag < (int64_t)T * B; ++bag) {
    const int t = (int)(bag / B);
    for (int64_t j = offsets[bag]; j < offsets[bag + 1]; ++j) {
      keys[j] = (uint64_t)(hash_size_cumsum[t] + indices[j]);
      pos[j] = (uint32_t)j;
      bag_of[j] = (int32_t)bag;
    }
  }
  int bits = 1;
  while (bits < 63 && ((uint64_t)hash_size_cumsum[T] >> bits) != 0) ++bits;
  sort_pairs(keys, pos, n, bits);

  /* segment starts */
  int64_t* seg = (int64_t*)malloc(sizeof(int64_t) * (size_t)(n + 1));
  int64_t nseg = 0;
  for (int64_t i = 0; i < n; ++i)
    if (i == 0 || keys[i] != keys[i - 1]) seg[nseg++] = i;
  seg[nseg] = n;

#pragma omp parallel for schedule(dynamic, 256)
  for (int64_t s = 0; s < nseg; ++s) {
    const uint64_t key = keys[seg[s]];
    int t = 0;
    while (t + 1 < T && (uint64_t)hash_size_cumsum[t + 1] <= key) ++t;
    const int64_t row = (int64_t)key - hash_size_cumsum[t];
    const int D = D_offsets[t + 1] - D_offsets[t];
    float g[4096];
    if (D > 4096) continue;
    for (int d = 0; d < D; ++d) g[d] = 0.f;
    for (int64_t i = seg[s]; i < seg[s + 1]; ++i) {
      const int64_t j = pos[i];
      const int64_t bag = bag_of[j];
      const int64_t b = bag % B;
      float w = per_sample_weights ? per_sample_weights[j] : 1.f;
      if (pooling_mode == POOL_MEAN) w /= (float)(offsets[bag + 1] - offsets[bag]);
      const float* gr = grad + b * grad_stride + D_offsets[t];
      for (int d = 0; d < D; ++d) g[d] += gr[d] * w;
    }
    float mult = lr;
    if (optimizer == OPT_ROWWISE_ADAGRAD) {
      float sq = 0.f;
      for (int d = 0; d < D; ++d) sq += g[d] * g[d];
      float* m = momentum1 + momentum1_offsets[t] + row;
      const float m_new = *m + sq / (float)D;
      *m = m_new;
      mult = lr / (sqrtf(m_new) + eps);
    }
    if (weights_ty == TY_FP32) {
      float* w = (float*)dev_weights + weights_offsets[t] + row * D;
      for (int d = 0; d < D; ++d) w[d] = w[d] - mult * g[d];
    } else {
      uint16_t* w = (uint16_t*)dev_weights + weights_offsets[t] + row * D;
      for (int d = 0; d < D; ++d)
        w[d] = oracle_float_to_half(oracle_half_to_float(w[d]) - mult * g[d]);
    }
  }
  free(seg);
  free(bag_of);
  free(pos);
  free(keys);
  return 0;
}

/* ---- jagged ops; elements are moved as elem_bytes-sized opaque items ----------------------- */
static int64_t jagged_row_of(const int64_t* const* offsets, const int64_t* max_lengths, int n,
                             int64_t total_rows, int64_t dense_row) {
  int64_t coord[8];
  int64_t r = dense_row;
  for (int d = n - 1; d >= 0; --d) {
    coord[d] = r % max_lengths[d];
    r /= max_lengths[d];
  }
  int64_t idx = r;
  for (int d = 0; d < n; ++d) {
    const int64_t begin = offsets[d][idx], end = offsets[d][idx + 1];
    if (coord[d] >= end - begin) return -1;
    idx = begin + coord[d];
  }
  return idx < total_rows ? idx : -1;
}

static int64_t dense_rows(int64_t outer, const int64_t* max_lengths, int n) {
  int64_t rows = outer;
  for (int d = 0; d < n; ++d) rows *= max_lengths[d];
  return rows;
}

ORACLE_API int oracle_jagged_to_padded_dense(const void* values, const int64_t* const* offsets,
                                             const int64_t* max_lengths, int n, int64_t outer,
                                             int64_t inner, int64_t total_rows, int elem_bytes,
                                             const void* pad_elem, void* dense) {
  if (n < 1 || n > 8) return -1;
  const int64_t rows = dense_rows(outer, max_lengths, n);
  const int64_t row_bytes = inner * elem_bytes;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    char* dst = (char*)dense + r * row_bytes;
    const int64_t src = jagged_row_of(offsets, max_lengths, n, total_rows, r);
    if (src >= 0) {
      memcpy(dst, (const char*)values + src * row_bytes, (size_t)row_bytes);
    } else {
      for (int64_t e = 0; e < inner; ++e) memcpy(dst + e * elem_bytes, pad_elem, (size_t)elem_bytes);
    }
  }
  return 0;
}

ORACLE_API int oracle_dense_to_jagged(const void* dense, const int64_t* const* offsets,
                                      const int64_t* max_lengths, int n, int64_t outer,
                                      int64_t inner, int64_t total_rows, int elem_bytes,
                                      void* values) {
  if (n < 1 || n > 8) return -1;
  const int64_t rows = dense_rows(outer, max_lengths, n);
  const int64_t row_bytes = inner * elem_bytes;
  memset(values, 0, (size_t)(total_rows * row_bytes));
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const int64_t dst = jagged_row_of(offsets, max_lengths, n, total_rows, r);
    if (dst >= 0)
      memcpy((char*)values + dst * row_bytes, (const char*)dense + r * row_bytes, (size_t)row_bytes);
  }
  return 0;
}

ORACLE_API int oracle_jagged_dense_elementwise_add_f32(const float* x_values,
                                                       const int64_t* const* offsets,
                                                       const int64_t* max_lengths, int n,
                                                       int64_t outer, int64_t inner,
                                                       int64_t total_rows, const float* y,
                                                       float* out) {
  if (n < 1 || n > 8) return -1;
  const int64_t rows = dense_rows(outer, max_lengths, n);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const int64_t src = jagged_row_of(offsets, max_lengths, n, total_rows, r);
    const float* yy = y + r * inner;
    float* o = out + r * inner;
    if (src >= 0) {
      const float* x = x_values + src * inner;
      for (int64_t e = 0; e < inner; ++e) o[e] = x[e] + yy[e];
    } else {
      for (int64_t e = 0; e < inner; ++e) o[e] = 0.f + yy[e];
    }
  }
  return 0;
}
