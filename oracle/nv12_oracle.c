/* CPU oracle of the NV12 -> RGB24 conversion: TEST INFRASTRUCTURE ONLY.
 *
 * Only tests/, __graft_entry__.smoke() and bench.py's CPU arms may load this library; the product
 * never does. It restates, in plain C with every floating-point operation spelled out (no
 * contraction: build with -ffp-contract=off), the arithmetic of the reference's only device kernel:
 *
 *   packages/torchcodec-xpu/src/torchcodec_xpu/ColorConversionKernel.cpp
 *     :12-16    BT.709 matrix rows {1, 0, 1.5748}, {1, -0.187324, -0.468124}, {1, 1.8556, 0}
 *     :29-80    byte offset of (x, y) in an Intel Tile-Y surface (128-byte x 32-row tiles, 16-byte
 *               columns, 64-byte halves swapped between neighbouring 4-row groups)
 *     :82-100   normalisation (limited range: (y-16)/219, (u-128)/224, (v-128)/224; "full range":
 *               y/255, (u-128)/255 - 0.5, (v-128)/255 - 0.5, as the reference writes it), the
 *               three dot products, x255, clamp to [0, 255], truncation to 8 bits
 *     :131-157  per pixel: chroma sample (x/2, y/2), U at byte 2*(x/2), V at the next byte, RGB
 *               packed at 3 * (y * width + x)
 *
 * Pin: the reference holds no test vectors for this kernel (its tests compare decoded frames by
 * PSNR against a CPU decoder that is not in the repository). The pins are (tests/test_nv12.py):
 * the reference's OWN source file compiled for the host (oracle/nv12_ref_wrap.cpp ->
 * oracle/_ref/libnv12_ref.so) -- its get_tile_offset over every byte of multi-tile surfaces, its
 * yuv2rgb over all 2^24 (y, u, v) triples in both range modes, its whole kernel over random Tile-Y
 * frames, all bit for bit -- and known answers of BT.709 itself: black, white, mid grey, primaries.
 *
 * The dot product is evaluated left to right, s0*m0 + s1*m1 + s2*m2, each product and sum rounded
 * to fp32; the CUDA kernel spells the same sequence with __fmul_rn / __fadd_rn. */
#include <stddef.h>
#include <stdint.h>

#define ORACLE_API __attribute__((visibility("default")))

static const float kBt709[3][3] = {
    {1.0f, 0.0f, 1.5748f},
    {1.0f, -0.187324f, -0.468124f},
    {1.0f, 1.8556f, 0.0f},
};

/* Byte offset of (x, y) in a surface of `stride` bytes per row; tiled = 1: Intel Tile-Y. */
ORACLE_API size_t nv12_oracle_offset(int x, int y, int stride, int tiled) {
  if (!tiled) return (size_t)y * (size_t)stride + (size_t)x;
  const int tile_col = x >> 7, tile_row = y >> 5;
  const int xi = x & 127, yi = y & 31;
  int half = xi >> 6;       /* which 64-byte half of the tile row */
  int group = yi >> 2;      /* which group of 4 rows */
  if ((half ^ group) & 1) { /* odd pairs sit in the other half of the neighbouring group */
    half ^= 1;
    group ^= 1;
  }
  const int column = half * 4 + ((xi & 63) >> 4); /* 16-byte column, 0..7 */
  const int in_tile = (group * 8 + column) * 64 + (yi & 3) * 16 + (xi & 15);
  return ((size_t)tile_row * (size_t)(stride >> 7) + (size_t)tile_col) * 4096u + (size_t)in_tile;
}

static uint8_t to_byte(float f) {
  float s = f * 255.0f;
  if (s < 0.0f) s = 0.0f;
  if (s > 255.0f) s = 255.0f;
  return (uint8_t)s;
}

ORACLE_API void nv12_oracle_pixel(uint8_t y, uint8_t u, uint8_t v, int fullrange, uint8_t* rgb) {
  float s0, s1, s2;
  if (fullrange) {
    s0 = (float)y / 255.0f;
    s1 = ((float)u - 128.0f) / 255.0f - 0.5f;
    s2 = ((float)v - 128.0f) / 255.0f - 0.5f;
  } else {
    s0 = ((float)y - 16.0f) / 219.0f;
    s1 = ((float)u - 128.0f) / 224.0f;
    s2 = ((float)v - 128.0f) / 224.0f;
  }
  for (int c = 0; c < 3; ++c) {
    float d = s0 * kBt709[c][0];
    d = d + s1 * kBt709[c][1];
    d = d + s2 * kBt709[c][2];
    rgb[c] = to_byte(d);
  }
}

/* out[3 * ((y << 16) | (u << 8) | v) ...] = RGB of the triple, for all 2^24 triples. */
ORACLE_API void nv12_oracle_all_triples(int fullrange, uint8_t* out) {
  for (int y = 0; y < 256; ++y)
    for (int u = 0; u < 256; ++u)
      for (int v = 0; v < 256; ++v)
        nv12_oracle_pixel((uint8_t)y, (uint8_t)u, (uint8_t)v, fullrange,
                          out + 3 * (((size_t)y << 16) | ((size_t)u << 8) | (size_t)v));
}

ORACLE_API void nv12_oracle_convert(const uint8_t* y_plane, const uint8_t* uv_plane, uint8_t* rgb,
                                    int width, int height, int stride, int fullrange, int tiled) {
  for (int yy = 0; yy < height; ++yy) {
    for (int xx = 0; xx < width; ++xx) {
      const int cx = xx >> 1, cy = yy >> 1;
      const uint8_t y = y_plane[nv12_oracle_offset(xx, yy, stride, tiled)];
      const uint8_t u = uv_plane[nv12_oracle_offset(2 * cx, cy, stride, tiled)];
      const uint8_t v = uv_plane[nv12_oracle_offset(2 * cx + 1, cy, stride, tiled)];
      nv12_oracle_pixel(y, u, v, fullrange, rgb + 3 * ((size_t)yy * (size_t)width + (size_t)xx));
    }
  }
}
