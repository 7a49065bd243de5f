// The reference's colour-conversion kernel itself, compiled for the host: TEST INFRASTRUCTURE ONLY.
//
// This file includes packages/torchcodec-xpu/src/torchcodec_xpu/ColorConversionKernel.cpp from the
// reference tree (found through the include path given by oracle/build.py; nothing of it is copied
// here) on top of oracle/sycl_host_shim, and exports its three functions with C linkage:
//   get_tile_offset   (ColorConversionKernel.cpp:29-80)
//   yuv2rgb           (:82-100), swept over every (y, u, v) triple
//   convertNV12ToRGB  (:160-181), the whole kernel over a Tile-Y surface
// tests/test_nv12.py pins oracle/nv12_oracle.c against them. The library is built only where the
// reference tree is present and travels as a built file.
#include <sycl/sycl.hpp>

#include "ColorConversionKernel.cpp"

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API size_t nv12_ref_tile_offset(int x, int y, int stride) {
  return facebook::torchcodec::get_tile_offset(x, y, stride);
}

// out[3 * ((y << 16) | (u << 8) | v) ...] = RGB of the triple, for all 2^24 triples.
REF_API void nv12_ref_all_triples(int fullrange, uint8_t* out) {
  for (int y = 0; y < 256; ++y)
    for (int u = 0; u < 256; ++u)
      for (int v = 0; v < 256; ++v) {
        const sycl::uchar3 rgb = facebook::torchcodec::yuv2rgb(
            static_cast<uint8_t>(y), static_cast<uint8_t>(u), static_cast<uint8_t>(v), fullrange != 0,
            facebook::torchcodec::rgb_matrix_bt709);
        uint8_t* o = out + 3 * ((static_cast<size_t>(y) << 16) | (static_cast<size_t>(u) << 8) | v);
        o[0] = rgb.x();
        o[1] = rgb.y();
        o[2] = rgb.z();
      }
}

REF_API void nv12_ref_convert(const uint8_t* y_plane, const uint8_t* uv_plane, uint8_t* rgb, int width,
                              int height, int stride, int fullrange) {
  sycl::queue q;
  facebook::torchcodec::convertNV12ToRGB(q, y_plane, uv_plane, rgb, width, height, stride, fullrange != 0);
}
