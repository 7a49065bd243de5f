// Row-wise min-max quantisation of fp32 / fp16 rows to INT8 / INT4 / INT2 with an fp16 {scale, bias}
// pair per row, and the inverse. One warp per row: the row is read with coalesced loads (a second
// time, out of L1 / L2, when it is packed), min and max are reduced by shuffle, scale = (max - bias) / (2^bits - 1) and bias = min are rounded to fp16 before they
// are used (what is stored is what dequantises), q = rint((x - bias) / scale) clamped. The header
// goes either in front of the payload (the TBE table layout, rows padded to row_alignment) or
// behind it (the layout of FBGEMM's fused N-bit row-wise ops). Streaming, HBM-bound.
#include "common.cuh"

namespace b200tbe {
namespace {

constexpr int kQWarps = 8;
constexpr int kQThreads = kQWarps * 32;

template <typename T>
__device__ __forceinline__ float load_elem(const T* p);
template <>
__device__ __forceinline__ float load_elem<float>(const float* p) {
  return __ldg(p);
}
template <>
__device__ __forceinline__ float load_elem<__half>(const __half* p) {
  return __half2float(__ldg(p));
}

struct QuantParams {
  const void* src;
  uint8_t* dst;
  int64_t rows;
  int32_t D;
  int32_t bits;
  int64_t dst_stride;
  int32_t header_first;
};

template <typename T>
__global__ void __launch_bounds__(kQThreads) quantize_rows_kernel(QuantParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kQWarps + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  const T* x = static_cast<const T*>(p.src) + row * p.D;
  uint8_t* out = p.dst + row * p.dst_stride;
  const int qmax = (1 << p.bits) - 1;
  const int per_byte = 8 / p.bits;
  const int payload = (p.D + per_byte - 1) / per_byte;
  uint8_t* body = out + (p.header_first ? 4 : 0);
  uint8_t* header = p.header_first ? out : out + payload;

  // each lane owns whole payload bytes: byte b = lane + 32*i, elements [b*per_byte, +per_byte)
  float mn = 3.4e38f, mx = -3.4e38f;
  for (int e = lane; e < p.D; e += 32) {
    const float v = load_elem<T>(x + e);
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(kFullMask, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(kFullMask, mx, o));
  }
  const __half hb = __float2half_rn(mn);
  const float bias = __half2float(hb);
  const float range = mx - bias;
  __half hs = __float2half_rn(range == 0.f ? 1.f : range / static_cast<float>(qmax));
  float scale = __half2float(hs);
  if (scale == 0.f) {  // range too small for fp16
    hs = __float2half_rn(1.f);
    scale = 1.f;
  }
  const float inv = 1.f / scale;
  for (int b = lane; b < payload; b += 32) {
    unsigned byte = 0;
    for (int k = 0; k < per_byte; ++k) {
      const int e = b * per_byte + k;
      if (e < p.D) {
        int q = __float2int_rn((load_elem<T>(x + e) - bias) * inv);
        q = q < 0 ? 0 : (q > qmax ? qmax : q);
        byte |= static_cast<unsigned>(q) << (k * p.bits);
      }
    }
    body[b] = static_cast<uint8_t>(byte);
  }
  if (lane == 0) {
    const unsigned short s = __half_as_ushort(hs), bb = __half_as_ushort(hb);
    header[0] = s & 0xff;
    header[1] = s >> 8;
    header[2] = bb & 0xff;
    header[3] = bb >> 8;
  }
  // zero the padding of aligned rows so that tables are reproducible byte for byte
  const int used = payload + 4;
  for (int64_t b = used + lane; b < p.dst_stride; b += 32) out[b] = 0;
}

struct DequantParams {
  const uint8_t* src;
  void* dst;
  int64_t rows;
  int32_t D;
  int32_t bits;
  int64_t src_stride;
  int32_t header_first;
};

template <typename T>
__global__ void __launch_bounds__(kQThreads) dequantize_rows_kernel(DequantParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kQWarps + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  const uint8_t* in = p.src + row * p.src_stride;
  const int per_byte = 8 / p.bits;
  const int payload = (p.D + per_byte - 1) / per_byte;
  const uint8_t* body = in + (p.header_first ? 4 : 0);
  const uint8_t* header = p.header_first ? in : in + payload;
  const unsigned s = header[0] | (header[1] << 8), b = header[2] | (header[3] << 8);
  const float scale = __half2float(__ushort_as_half(static_cast<unsigned short>(s)));
  const float bias = __half2float(__ushort_as_half(static_cast<unsigned short>(b)));
  T* y = static_cast<T*>(p.dst) + row * p.D;
  const unsigned mask = (1u << p.bits) - 1u;
  for (int e = lane; e < p.D; e += 32) {
    const unsigned q = (body[e / per_byte] >> ((e % per_byte) * p.bits)) & mask;
    const float v = fmaf(static_cast<float>(q), scale, bias);
    if (sizeof(T) == 4) {
      reinterpret_cast<float*>(y)[e] = v;
    } else {
      reinterpret_cast<__half*>(y)[e] = __float2half_rn(v);
    }
  }
}

// ---- vector paths: D a multiple of 4, at most 512, aligned rows -----------------------------------
// A lane owns whole groups of four elements (group j = v * 32 + lane, v < V): one 16-byte (fp32) or
// 8-byte (fp16) load per group, so the row lives in registers and is read once; the four codes of a
// group are one 32-, 16- or 8-bit store. A warp keeps 4 / V rows in flight. Same arithmetic, in the
// same order per element, as the scalar kernels above.
template <typename T>
__device__ __forceinline__ float4 load_group(const T* p);
template <>
__device__ __forceinline__ float4 load_group<float>(const float* p) {
  return __ldg(reinterpret_cast<const float4*>(p));
}
template <>
__device__ __forceinline__ float4 load_group<__half>(const __half* p) {
  const uint2 r = __ldg(reinterpret_cast<const uint2*>(p));
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

template <typename T, int V>
__global__ void __launch_bounds__(kQThreads) quantize_rows_vec_kernel(QuantParams p) {
  constexpr int R = 4 / V;
  const int lane = threadIdx.x & 31;
  const int64_t row0 = (static_cast<int64_t>(blockIdx.x) * kQWarps + (threadIdx.x >> 5)) * R;
  if (row0 >= p.rows) return;
  const int qmax = (1 << p.bits) - 1;
  const int payload = p.D * p.bits / 8;
  float4 x[R][V];
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int v = 0; v < V; ++v) {
      const int j = v * 32 + lane;
      x[r][v] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row0 + r < p.rows && 4 * j < p.D)
        x[r][v] = load_group<T>(static_cast<const T*>(p.src) + (row0 + r) * p.D + 4 * j);
    }
  }
  // the R rows' reductions run side by side (each is a chain of dependent shuffles)
  float mn[R], mx[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    mn[r] = 3.4e38f;
    mx[r] = -3.4e38f;
#pragma unroll
    for (int v = 0; v < V; ++v) {
      if (4 * (v * 32 + lane) < p.D) {
        mn[r] = fminf(fminf(mn[r], x[r][v].x), fminf(fminf(x[r][v].y, x[r][v].z), x[r][v].w));
        mx[r] = fmaxf(fmaxf(mx[r], x[r][v].x), fmaxf(fmaxf(x[r][v].y, x[r][v].z), x[r][v].w));
      }
    }
  }
  // R rows' minima and maxima across the warp. Reducing them one by one takes 10 shuffles a row;
  // instead the lanes split the rows between them as they go: after the exchange over 16 lanes each
  // half-warp carries half of the rows, after the one over 8 lanes (four rows) each quarter one row,
  // and the remaining exchanges finish that row. Row r ends up in the lanes whose index / 8 (four
  // rows) or / 16 (two rows) is r.
  float my_mn, my_mx;
  int my_row;     // the row whose extremes this lane ends up with
  if constexpr (R == 4) {
    const bool hi16 = lane & 16, hi8 = lane & 8;
    float a[2], b2[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float omn = __shfl_xor_sync(kFullMask, hi16 ? mn[i] : mn[i + 2], 16);
      const float omx = __shfl_xor_sync(kFullMask, hi16 ? mx[i] : mx[i + 2], 16);
      a[i] = fminf(hi16 ? mn[i + 2] : mn[i], omn);
      b2[i] = fmaxf(hi16 ? mx[i + 2] : mx[i], omx);
    }
    const float omn = __shfl_xor_sync(kFullMask, hi8 ? a[0] : a[1], 8);
    const float omx = __shfl_xor_sync(kFullMask, hi8 ? b2[0] : b2[1], 8);
    my_mn = fminf(hi8 ? a[1] : a[0], omn);
    my_mx = fmaxf(hi8 ? b2[1] : b2[0], omx);
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      my_mn = fminf(my_mn, __shfl_xor_sync(kFullMask, my_mn, o));
      my_mx = fmaxf(my_mx, __shfl_xor_sync(kFullMask, my_mx, o));
    }
    my_row = lane >> 3;
  } else if constexpr (R == 2) {
    const bool hi16 = lane & 16;
    const float omn = __shfl_xor_sync(kFullMask, hi16 ? mn[0] : mn[1], 16);
    const float omx = __shfl_xor_sync(kFullMask, hi16 ? mx[0] : mx[1], 16);
    my_mn = fminf(hi16 ? mn[1] : mn[0], omn);
    my_mx = fmaxf(hi16 ? mx[1] : mx[0], omx);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
      my_mn = fminf(my_mn, __shfl_xor_sync(kFullMask, my_mn, o));
      my_mx = fmaxf(my_mx, __shfl_xor_sync(kFullMask, my_mx, o));
    }
    my_row = lane >> 4;
  } else {
    my_mn = mn[0];
    my_mx = mx[0];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      my_mn = fminf(my_mn, __shfl_xor_sync(kFullMask, my_mn, o));
      my_mx = fmaxf(my_mx, __shfl_xor_sync(kFullMask, my_mx, o));
    }
    my_row = 0;
  }
  constexpr int kLanesPerRow = 32 / R;   // lane r * kLanesPerRow is the first that holds row r's scalars
  // The per-row scalars (fp16 bias and scale, the reciprocal) cost as many instructions for one
  // lane as for 32: every lane works them out for the row it holds and hands them round; the first
  // lane of a row's share also writes its header.
  const __half hb = __float2half_rn(my_mn);
  const float my_bias = __half2float(hb);
  const float range = my_mx - my_bias;
  __half hs = __float2half_rn(range == 0.f ? 1.f : range / static_cast<float>(qmax));
  float my_scale = __half2float(hs);
  if (my_scale == 0.f) {  // range too small for fp16
    hs = __float2half_rn(1.f);
    my_scale = 1.f;
  }
  const float my_inv = 1.f / my_scale;
  const uint32_t my_header = static_cast<uint32_t>(__half_as_ushort(hs)) | (static_cast<uint32_t>(__half_as_ushort(hb)) << 16);
  // header and padding as whole words where the row's layout allows it
  const bool words = (payload & 3) == 0;
  if ((lane & (kLanesPerRow - 1)) == 0 && row0 + my_row < p.rows) {
    uint8_t* out = p.dst + (row0 + my_row) * p.dst_stride;
    uint8_t* header = p.header_first ? out : out + payload;
    if (words) {
      *reinterpret_cast<uint32_t*>(header) = my_header;
    } else {
      header[0] = my_header & 0xff;
      header[1] = (my_header >> 8) & 0xff;
      header[2] = (my_header >> 16) & 0xff;
      header[3] = my_header >> 24;
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const float bias = __shfl_sync(kFullMask, my_bias, r * kLanesPerRow);
    const float inv = __shfl_sync(kFullMask, my_inv, r * kLanesPerRow);
    if (row0 + r >= p.rows) continue;
    uint8_t* out = p.dst + (row0 + r) * p.dst_stride;
    uint8_t* body = out + (p.header_first ? 4 : 0);
#pragma unroll
    for (int v = 0; v < V; ++v) {
      const int j = v * 32 + lane;
      if (4 * j >= p.D) continue;
      const float e[4] = {x[r][v].x, x[r][v].y, x[r][v].z, x[r][v].w};
      unsigned word = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        // round to nearest even; the conversion saturates at 0 and 255 (and turns NaN into 0), as
        // __float2int_rn followed by the clamp does
        unsigned q;
        asm("cvt.rni.u8.f32 %0, %1;" : "=r"(q) : "f"((e[k] - bias) * inv));
        q = q > static_cast<unsigned>(qmax) ? static_cast<unsigned>(qmax) : q;
        word |= q << (k * p.bits);
      }
      if (p.bits == 8) {
        *reinterpret_cast<uint32_t*>(body + 4 * j) = word;
      } else if (p.bits == 4) {
        *reinterpret_cast<uint16_t*>(body + 2 * j) = static_cast<uint16_t>(word);
      } else {
        body[j] = static_cast<uint8_t>(word);
      }
    }
    // the padding of aligned rows is zeroed so that tables are reproducible byte for byte
    if (words) {
      const int pad_words = static_cast<int>(p.dst_stride - payload - 4) >> 2;
      for (int w = lane; w < pad_words; w += 32) *reinterpret_cast<uint32_t*>(out + payload + 4 + 4 * w) = 0u;
    } else {
      for (int64_t b2 = payload + 4 + lane; b2 < p.dst_stride; b2 += 32) out[b2] = 0;
    }
  }
}

template <typename T>
__device__ __forceinline__ void store_group(T* p, float4 v);
template <>
__device__ __forceinline__ void store_group<float>(float* p, float4 v) {
  *reinterpret_cast<float4*>(p) = v;
}
template <>
__device__ __forceinline__ void store_group<__half>(__half* p, float4 v) {
  const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

template <typename T, int V>
__global__ void __launch_bounds__(kQThreads) dequantize_rows_vec_kernel(DequantParams p) {
  constexpr int R = 4 / V;
  const int lane = threadIdx.x & 31;
  const int64_t row0 = (static_cast<int64_t>(blockIdx.x) * kQWarps + (threadIdx.x >> 5)) * R;
  if (row0 >= p.rows) return;
  const int payload = p.D * p.bits / 8;
  const unsigned mask = (1u << p.bits) - 1u;
  unsigned word[R][V];
  unsigned hdr[R];                 // {scale, bias} as stored: two fp16
  const bool header_word = p.header_first || (payload & 3) == 0;   // the header is 4-byte aligned
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint8_t* in = p.src + (row0 + r) * p.src_stride;
    const uint8_t* body = in + (p.header_first ? 4 : 0);
    const uint8_t* header = p.header_first ? in : in + payload;
    const bool live = row0 + r < p.rows;
    hdr[r] = 0u;
    if (live) {
      if (header_word) {
        hdr[r] = __ldg(reinterpret_cast<const uint32_t*>(header));
      } else {
        hdr[r] = header[0] | (header[1] << 8) | (header[2] << 16) | (static_cast<unsigned>(header[3]) << 24);
      }
    }
#pragma unroll
    for (int v = 0; v < V; ++v) {
      const int j = v * 32 + lane;
      word[r][v] = 0;
      if (live && 4 * j < p.D) {
        if (p.bits == 8) {
          word[r][v] = __ldg(reinterpret_cast<const uint32_t*>(body + 4 * j));
        } else if (p.bits == 4) {
          word[r][v] = __ldg(reinterpret_cast<const uint16_t*>(body + 2 * j));
        } else {
          word[r][v] = __ldg(body + j);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (row0 + r >= p.rows) break;
    const float scale = __half2float(__ushort_as_half(static_cast<unsigned short>(hdr[r] & 0xffffu)));
    const float bias = __half2float(__ushort_as_half(static_cast<unsigned short>(hdr[r] >> 16)));
    T* y = static_cast<T*>(p.dst) + (row0 + r) * p.D;
#pragma unroll
    for (int v = 0; v < V; ++v) {
      const int j = v * 32 + lane;
      if (4 * j >= p.D) continue;
      const unsigned w = word[r][v];
      store_group<T>(y + 4 * j, make_float4(fmaf(static_cast<float>(w & mask), scale, bias),
                                            fmaf(static_cast<float>((w >> p.bits) & mask), scale, bias),
                                            fmaf(static_cast<float>((w >> (2 * p.bits)) & mask), scale, bias),
                                            fmaf(static_cast<float>((w >> (3 * p.bits)) & mask), scale, bias)));
    }
  }
}

// The vector paths want whole groups of four elements, rows of at most 512 elements, and pointers and
// row pitches that keep every group's load and store aligned.
bool vector_path_ok(const void* matrix, int elem_bytes, const uint8_t* quantised, int64_t q_stride, int32_t D) {
  if ((D & 3) != 0 || D > 512) return false;
  if ((reinterpret_cast<uintptr_t>(matrix) & (4 * elem_bytes - 1)) != 0) return false;
  return (reinterpret_cast<uintptr_t>(quantised) & 3) == 0 && (q_stride & 3) == 0;
}

int bits_of(int ty) {
  switch (ty) {
    case B200TBE_INT8: return 8;
    case B200TBE_INT4: return 4;
    case B200TBE_INT2: return 2;
    default: return 0;
  }
}

}  // namespace
}  // namespace b200tbe

using namespace b200tbe;

extern "C" int64_t b200tbe_quantized_row_bytes(int32_t D, int32_t ty, int32_t row_alignment) {
  const int bits = bits_of(ty);
  if (bits == 0 || D < 0 || row_alignment < 1) return -1;
  const int64_t bytes = 4 + (static_cast<int64_t>(D) * bits + 7) / 8;
  return (bytes + row_alignment - 1) / row_alignment * row_alignment;
}

extern "C" int b200tbe_quantize_rows(const void* src, int32_t src_dtype, int64_t rows, int32_t D,
                                     int32_t ty, int32_t row_alignment, int32_t header_first,
                                     uint8_t* dst, b200tbe_stream_t stream_) {
  const int bits = bits_of(ty);
  if (bits == 0) return B200TBE_ERR_UNSUPPORTED;
  if (rows < 0 || D < 0 || row_alignment < 1) return B200TBE_ERR_BAD_ARG;
  if (rows == 0 || D == 0) return B200TBE_OK;
  if (src == nullptr || dst == nullptr) return B200TBE_ERR_BAD_ARG;
  const int64_t ctas = (rows + kQWarps - 1) / kQWarps;
  if (ctas > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  QuantParams p{src, dst, rows, D, bits, b200tbe_quantized_row_bytes(D, ty, row_alignment),
                header_first};
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (src_dtype != B200TBE_FP32 && src_dtype != B200TBE_FP16) return B200TBE_ERR_UNSUPPORTED;
  const bool f32 = src_dtype == B200TBE_FP32;
  // payload groups must be aligned too: with the header in front they start 4 bytes into the row
  if (vector_path_ok(src, f32 ? 4 : 2, dst, p.dst_stride, D)) {
    const int V = D <= 128 ? 1 : (D <= 256 ? 2 : 4);
    const unsigned grid = static_cast<unsigned>((rows + kQWarps * (4 / V) - 1) / (kQWarps * (4 / V)));
    if (f32) {
      if (V == 1) quantize_rows_vec_kernel<float, 1><<<grid, kQThreads, 0, stream>>>(p);
      else if (V == 2) quantize_rows_vec_kernel<float, 2><<<grid, kQThreads, 0, stream>>>(p);
      else quantize_rows_vec_kernel<float, 4><<<grid, kQThreads, 0, stream>>>(p);
    } else {
      if (V == 1) quantize_rows_vec_kernel<__half, 1><<<grid, kQThreads, 0, stream>>>(p);
      else if (V == 2) quantize_rows_vec_kernel<__half, 2><<<grid, kQThreads, 0, stream>>>(p);
      else quantize_rows_vec_kernel<__half, 4><<<grid, kQThreads, 0, stream>>>(p);
    }
    return launch_status();
  }
  if (f32) {
    quantize_rows_kernel<float><<<static_cast<unsigned>(ctas), kQThreads, 0, stream>>>(p);
  } else {
    quantize_rows_kernel<__half><<<static_cast<unsigned>(ctas), kQThreads, 0, stream>>>(p);
  }
  return launch_status();
}

extern "C" int b200tbe_dequantize_rows(const uint8_t* src, int64_t rows, int32_t D, int32_t ty,
                                       int32_t row_alignment, int32_t header_first, void* dst,
                                       int32_t dst_dtype, b200tbe_stream_t stream_) {
  const int bits = bits_of(ty);
  if (bits == 0) return B200TBE_ERR_UNSUPPORTED;
  if (rows < 0 || D < 0 || row_alignment < 1) return B200TBE_ERR_BAD_ARG;
  if (rows == 0 || D == 0) return B200TBE_OK;
  if (src == nullptr || dst == nullptr) return B200TBE_ERR_BAD_ARG;
  const int64_t ctas = (rows + kQWarps - 1) / kQWarps;
  if (ctas > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
  DequantParams p{src, dst, rows, D, bits, b200tbe_quantized_row_bytes(D, ty, row_alignment),
                  header_first};
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (dst_dtype != B200TBE_FP32 && dst_dtype != B200TBE_FP16) return B200TBE_ERR_UNSUPPORTED;
  const bool f32 = dst_dtype == B200TBE_FP32;
  if (vector_path_ok(dst, f32 ? 4 : 2, src, p.src_stride, D)) {
    const int V = D <= 128 ? 1 : (D <= 256 ? 2 : 4);
    const unsigned grid = static_cast<unsigned>((rows + kQWarps * (4 / V) - 1) / (kQWarps * (4 / V)));
    if (f32) {
      if (V == 1) dequantize_rows_vec_kernel<float, 1><<<grid, kQThreads, 0, stream>>>(p);
      else if (V == 2) dequantize_rows_vec_kernel<float, 2><<<grid, kQThreads, 0, stream>>>(p);
      else dequantize_rows_vec_kernel<float, 4><<<grid, kQThreads, 0, stream>>>(p);
    } else {
      if (V == 1) dequantize_rows_vec_kernel<__half, 1><<<grid, kQThreads, 0, stream>>>(p);
      else if (V == 2) dequantize_rows_vec_kernel<__half, 2><<<grid, kQThreads, 0, stream>>>(p);
      else dequantize_rows_vec_kernel<__half, 4><<<grid, kQThreads, 0, stream>>>(p);
    }
    return launch_status();
  }
  if (f32) {
    dequantize_rows_kernel<float><<<static_cast<unsigned>(ctas), kQThreads, 0, stream>>>(p);
  } else {
    dequantize_rows_kernel<__half><<<static_cast<unsigned>(ctas), kQThreads, 0, stream>>>(p);
  }
  return launch_status();
}
