// NV12 -> packed RGB24 (BT.709), the one device kernel the reference plugin ships
// (packages/torchcodec-xpu/src/torchcodec_xpu/ColorConversionKernel.cpp:102-181), for B200.
//
// Byte work bound by HBM: 1.5 bytes read and 3 written per pixel. The reference runs one work-item
// per pixel with three single-byte loads and three single-byte stores; here a thread owns a block of
// 16 pixels x 2 rows: one 16-byte load per luma row, one 16-byte load of the shared chroma row, and
// three 16-byte stores per output row, all aligned, so a warp moves whole 128-byte lines. A 16-byte
// column is contiguous in both surface layouts (linear pitch and Intel Tile-Y, whose unit is the
// 16-byte OWord), only its address differs. Frames whose width is not a multiple of 16, or whose
// pointers / pitch are not 16-byte aligned, take a one-thread-per-pixel path.
//
// Arithmetic: every fp32 operation is issued with an explicit round-to-nearest intrinsic in the
// order the CPU oracle uses, so the two agree bit for bit. The divisions of the normalisation would
// make the kernel issue-bound (about 67 instructions per pixel measured). Their dividends are bytes,
// though, and for a byte the quotient equals one refinement step on the product with the rounded
// reciprocal (two fused multiply-adds, exact for all 256 values: luma_of, chroma_of), so the block
// path divides nothing; tables of the one-byte terms in shared memory, the version before this one,
// were bound by bank conflicts on random pixels (16.5 us per 4K frame against 12.6).
#include "common.cuh"

namespace b200tbe {
namespace {

constexpr int kNv12Threads = 256;

// Byte offset of (x, y) in a surface of `stride` bytes per row. Tile-Y: 128-byte x 32-row tiles of
// 4 KB, stored as 16-byte columns of 4 rows; the two 64-byte halves trade places between
// neighbouring 4-row groups (ColorConversionKernel.cpp:29-80).
__device__ __forceinline__ size_t surface_offset(int x, int y, int stride, bool tiled) {
  if (!tiled) return static_cast<size_t>(y) * static_cast<size_t>(stride) + static_cast<size_t>(x);
  const int xi = x & 127, yi = y & 31;
  int half = xi >> 6, group = yi >> 2;
  const int odd = (half ^ group) & 1;
  half ^= odd;
  group ^= odd;
  const int column = half * 4 + ((xi & 63) >> 4);
  const int in_tile = (group * 8 + column) * 64 + (yi & 3) * 16 + (xi & 15);
  return (static_cast<size_t>(y >> 5) * static_cast<size_t>(stride >> 7) + static_cast<size_t>(x >> 7)) * 4096u +
         static_cast<size_t>(in_tile);
}

struct Chroma {
  float s1, s2;
};

__device__ __forceinline__ Chroma chroma_terms(uint32_t u, uint32_t v, bool fullrange) {
  Chroma c;
  if (fullrange) {
    c.s1 = __fsub_rn(__fdiv_rn(__fsub_rn(static_cast<float>(u), 128.0f), 255.0f), 0.5f);
    c.s2 = __fsub_rn(__fdiv_rn(__fsub_rn(static_cast<float>(v), 128.0f), 255.0f), 0.5f);
  } else {
    c.s1 = __fdiv_rn(__fsub_rn(static_cast<float>(u), 128.0f), 224.0f);
    c.s2 = __fdiv_rn(__fsub_rn(static_cast<float>(v), 128.0f), 224.0f);
  }
  return c;
}

__device__ __forceinline__ uint32_t to_byte(float f) {
  const float s = fminf(fmaxf(__fmul_rn(f, 255.0f), 0.0f), 255.0f);
  return __float2uint_rz(s);
}

// {R, G, B} of one pixel (ColorConversionKernel.cpp:12-16, 82-100): rows {1, 0, 1.5748},
// {1, -0.187324, -0.468124}, {1, 1.8556, 0}; each dot product left to right.
__device__ __forceinline__ void pixel_rgb(uint32_t y, Chroma c, bool fullrange, uint32_t (&rgb)[3]) {
  const float s0 = fullrange ? __fdiv_rn(static_cast<float>(y), 255.0f)
                             : __fdiv_rn(__fsub_rn(static_cast<float>(y), 16.0f), 219.0f);
  const float m1[3] = {0.0f, -0.187324f, 1.8556f};
  const float m2[3] = {1.5748f, -0.468124f, 0.0f};
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    float d = __fmul_rn(s0, 1.0f);
    d = __fadd_rn(d, __fmul_rn(c.s1, m1[k]));
    d = __fadd_rn(d, __fmul_rn(c.s2, m2[k]));
    rgb[k] = to_byte(d);
  }
}

// Byte i of the vector as the float 2^23 + byte: the byte dropped into the mantissa of 8388608.0 by one
// permute (exact; the caller subtracts 2^23 together with its own offset).
__device__ __forceinline__ float byte_plus_2p23(uint4 v, int i) {
  const uint32_t w = i < 4 ? v.x : (i < 8 ? v.y : (i < 12 ? v.z : v.w));
  return __uint_as_float(__byte_perm(w, 0x4b000000u, 0x7540u + (i & 3)));
}

// x * 255 truncated to a byte; the conversion saturates at 0 and 255, which is the clamp.
__device__ __forceinline__ uint32_t to_byte_sat(float f) {
  uint32_t r;
  asm("cvt.rzi.u8.f32 %0, %1;" : "=r"(r) : "f"(__fmul_rn(f, 255.0f)));
  return r;
}

// The normalised luma without a table and without a division: (y - sub) / div for a byte y equals, bit
// for bit, one refinement step on the product with the rounded reciprocal -- q0 = a * r,
// q = fma(fma(-q0, div, a), r, q0) -- for all 256 bytes and both ranges (checked exhaustively on the
// host against IEEE division; the bit-exact tests against the reference's kernel cover it again).
struct LumaScale {
  float sub, div, recip;
};
__device__ __forceinline__ float luma_of(float y_plus_2p23, const LumaScale& k) {
  const float a = __fsub_rn(y_plus_2p23, 8388608.0f + k.sub);      // both exact
  const float q0 = __fmul_rn(a, k.recip);
  return __fmaf_rn(__fmaf_rn(-q0, k.div, a), k.recip, q0);
}

// The same for a chroma byte: (c - 128) / 224, or in the reference's "full range" branch
// (c - 128) / 255 - 0.5.
__device__ __forceinline__ float chroma_of(float c_plus_2p23, const LumaScale& k) {
  const float a = __fsub_rn(c_plus_2p23, 8388608.0f + 128.0f);
  const float q0 = __fmul_rn(a, k.recip);
  const float q = __fmaf_rn(__fmaf_rn(-q0, k.div, a), k.recip, q0);
  return __fsub_rn(q, k.sub);      // sub is 0 or 0.5: subtracting +0 changes nothing
}

// 16 pixels of one row -> 48 bytes, three aligned 16-byte stores.
__device__ __forceinline__ void convert_row16(const LumaScale& ls, const LumaScale& cs, uint4 luma, uint4 chroma,
                                              uint8_t* dst) {
  uint32_t bytes[48];
#pragma unroll
  for (int pair = 0; pair < 8; ++pair) {
    // {U into G, U into B} and {V into R, V into G}; the products with the matrix's zeros are +-0 and
    // adding them changes nothing
    const float cu = chroma_of(byte_plus_2p23(chroma, 2 * pair), cs), cv = chroma_of(byte_plus_2p23(chroma, 2 * pair + 1), cs);
    const float2 fu = make_float2(__fmul_rn(cu, -0.187324f), __fmul_rn(cu, 1.8556f));
    const float2 fv = make_float2(__fmul_rn(cv, 1.5748f), __fmul_rn(cv, -0.468124f));
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const float s0 = luma_of(byte_plus_2p23(luma, 2 * pair + s), ls);
      bytes[3 * (2 * pair + s) + 0] = to_byte_sat(__fadd_rn(s0, fv.x));
      bytes[3 * (2 * pair + s) + 1] = to_byte_sat(__fadd_rn(__fadd_rn(s0, fu.x), fv.y));
      bytes[3 * (2 * pair + s) + 2] = to_byte_sat(__fadd_rn(s0, fu.y));
    }
  }
  uint32_t w[12];
#pragma unroll
  for (int j = 0; j < 12; ++j)
    w[j] = bytes[4 * j] | (bytes[4 * j + 1] << 8) | (bytes[4 * j + 2] << 16) | (bytes[4 * j + 3] << 24);
  uint4* out = reinterpret_cast<uint4*>(dst);
  out[0] = make_uint4(w[0], w[1], w[2], w[3]);
  out[1] = make_uint4(w[4], w[5], w[6], w[7]);
  out[2] = make_uint4(w[8], w[9], w[10], w[11]);
}

// A plain grid, one block of 16 pixels x 2 rows per thread, no shared memory.
__global__ void __launch_bounds__(kNv12Threads)
    nv12_to_rgb_blocks_kernel(const uint8_t* __restrict__ y_plane, const uint8_t* __restrict__ uv_plane,
                              uint8_t* __restrict__ rgb, int width, int height, int stride,
                              bool fullrange, bool tiled) {
  const int groups = width >> 4;                 // 16-pixel blocks per row
  const int64_t block = static_cast<int64_t>(blockIdx.x) * kNv12Threads + threadIdx.x;
  const int64_t total = static_cast<int64_t>(groups) * ((height + 1) >> 1);
  const bool mine = block < total;
  const int gy = mine ? static_cast<int>(block / groups) : 0;
  const int x = mine ? static_cast<int>(block - static_cast<int64_t>(gy) * groups) << 4 : 0;
  const int y0 = gy * 2;
  const bool second = mine && y0 + 1 < height;
  uint4 chroma = make_uint4(0u, 0u, 0u, 0u), luma0 = chroma, luma1 = chroma;
  if (mine) {
    chroma = ldg_stream16(uv_plane + surface_offset(x, gy, stride, tiled));
    luma0 = ldg_stream16(y_plane + surface_offset(x, y0, stride, tiled));
  }
  if (second) luma1 = ldg_stream16(y_plane + surface_offset(x, y0 + 1, stride, tiled));
  const LumaScale ls = fullrange ? LumaScale{0.0f, 255.0f, __fdiv_rn(1.0f, 255.0f)}
                                 : LumaScale{16.0f, 219.0f, __fdiv_rn(1.0f, 219.0f)};
  const LumaScale cs = fullrange ? LumaScale{0.5f, 255.0f, __fdiv_rn(1.0f, 255.0f)}
                                 : LumaScale{0.0f, 224.0f, __fdiv_rn(1.0f, 224.0f)};
  if (mine) convert_row16(ls, cs, luma0, chroma, rgb + 3 * (static_cast<size_t>(y0) * width + x));
  if (second) convert_row16(ls, cs, luma1, chroma, rgb + 3 * (static_cast<size_t>(y0 + 1) * width + x));
}

__global__ void __launch_bounds__(kNv12Threads)
    nv12_to_rgb_pixels_kernel(const uint8_t* __restrict__ y_plane, const uint8_t* __restrict__ uv_plane,
                              uint8_t* __restrict__ rgb, int width, int height, int stride,
                              bool fullrange, bool tiled) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * kNv12Threads + threadIdx.x;
  if (i >= static_cast<int64_t>(width) * height) return;
  const int yy = static_cast<int>(i / width);
  const int xx = static_cast<int>(i - static_cast<int64_t>(yy) * width);
  const int cx = xx >> 1, cy = yy >> 1;
  const uint32_t y = y_plane[surface_offset(xx, yy, stride, tiled)];
  const uint32_t u = uv_plane[surface_offset(2 * cx, cy, stride, tiled)];
  const uint32_t v = uv_plane[surface_offset(2 * cx + 1, cy, stride, tiled)];
  uint32_t out[3];
  pixel_rgb(y, chroma_terms(u, v, fullrange), fullrange, out);
  uint8_t* dst = rgb + 3 * static_cast<size_t>(i);
  dst[0] = static_cast<uint8_t>(out[0]);
  dst[1] = static_cast<uint8_t>(out[1]);
  dst[2] = static_cast<uint8_t>(out[2]);
}

}  // namespace
}  // namespace b200tbe

using namespace b200tbe;

extern "C" int b200tbe_nv12_to_rgb(const uint8_t* y_plane, const uint8_t* uv_plane, uint8_t* rgb,
                                   int32_t width, int32_t height, int32_t stride, int32_t fullrange,
                                   int32_t tiled, b200tbe_stream_t stream_) {
  if (width < 0 || height < 0) return B200TBE_ERR_BAD_ARG;
  if (width == 0 || height == 0) return B200TBE_OK;
  if (y_plane == nullptr || uv_plane == nullptr || rgb == nullptr) return B200TBE_ERR_BAD_ARG;
  if (stride < width + (width & 1)) return B200TBE_ERR_BAD_ARG;   // a chroma pair must fit the row
  if (tiled != 0 && (stride & 127) != 0) return B200TBE_ERR_BAD_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const bool aligned = (width & 15) == 0 && (stride & 15) == 0 &&
                       ((reinterpret_cast<uintptr_t>(y_plane) | reinterpret_cast<uintptr_t>(uv_plane) |
                         reinterpret_cast<uintptr_t>(rgb)) & 15) == 0;
  if (aligned) {
    const int64_t blocks = static_cast<int64_t>(width >> 4) * ((height + 1) >> 1);
    const int64_t ctas = (blocks + kNv12Threads - 1) / kNv12Threads;
    if (ctas > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
    nv12_to_rgb_blocks_kernel<<<static_cast<unsigned>(ctas), kNv12Threads, 0, stream>>>(
        y_plane, uv_plane, rgb, width, height, stride, fullrange != 0, tiled != 0);
  } else {
    const int64_t ctas = (static_cast<int64_t>(width) * height + kNv12Threads - 1) / kNv12Threads;
    if (ctas > 0x7fffffff) return B200TBE_ERR_TOO_LARGE;
    nv12_to_rgb_pixels_kernel<<<static_cast<unsigned>(ctas), kNv12Threads, 0, stream>>>(
        y_plane, uv_plane, rgb, width, height, stride, fullrange != 0, tiled != 0);
  }
  return launch_status();
}
