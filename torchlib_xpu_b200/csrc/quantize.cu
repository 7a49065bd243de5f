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
  if (src_dtype == B200TBE_FP32) {
    quantize_rows_kernel<float><<<static_cast<unsigned>(ctas), kQThreads, 0, stream>>>(p);
  } else if (src_dtype == B200TBE_FP16) {
    quantize_rows_kernel<__half><<<static_cast<unsigned>(ctas), kQThreads, 0, stream>>>(p);
  } else {
    return B200TBE_ERR_UNSUPPORTED;
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
  if (dst_dtype == B200TBE_FP32) {
    dequantize_rows_kernel<float><<<static_cast<unsigned>(ctas), kQThreads, 0, stream>>>(p);
  } else if (dst_dtype == B200TBE_FP16) {
    dequantize_rows_kernel<__half><<<static_cast<unsigned>(ctas), kQThreads, 0, stream>>>(p);
  } else {
    return B200TBE_ERR_UNSUPPORTED;
  }
  return launch_status();
}
