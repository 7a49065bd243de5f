// Host stand-in for the few SYCL names the reference's colour-conversion kernel uses, so that the
// reference's own source file compiles with g++ and runs on the CPU: TEST INFRASTRUCTURE ONLY.
//
// It lets oracle/nv12_ref_wrap.cpp compile
//   packages/torchcodec-xpu/src/torchcodec_xpu/ColorConversionKernel.cpp
// unchanged, from where it lies in the reference tree. What the stand-in decides, and SYCL leaves to
// the device compiler, is how sycl::dot rounds: here a*x + b*y + c*z evaluated left to right in
// fp32; whether products and sums are contracted into fused multiply-adds is the C++ compiler's
// choice (-ffp-contract), and the build makes one library of each kind.
#pragma once

#include <array>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <utility>

namespace sycl {

template <typename T>
class vec3 {
 public:
  vec3() : v_{T(), T(), T()} {}
  vec3(T a, T b, T c) : v_{a, b, c} {}
  T& x() { return v_[0]; }
  T& y() { return v_[1]; }
  T& z() { return v_[2]; }
  const T& x() const { return v_[0]; }
  const T& y() const { return v_[1]; }
  const T& z() const { return v_[2]; }
  T& operator[](int i) { return v_[i]; }
  const T& operator[](int i) const { return v_[i]; }

 private:
  T v_[3];
};
using float3 = vec3<float>;
using uchar3 = vec3<std::uint8_t>;

inline float dot(const float3& a, const float3& b) {
  float d = a.x() * b.x();
  d = d + a.y() * b.y();
  d = d + a.z() * b.z();
  return d;
}

inline double floor(double v) { return std::floor(v); }

template <int N>
class id {
 public:
  id(std::size_t a, std::size_t b) : v_{a, b} {}
  std::size_t operator[](int i) const { return v_[i]; }

 private:
  std::size_t v_[N];
};

template <int N>
class range {
 public:
  range(std::size_t a, std::size_t b) : v_{a, b} {}
  std::size_t operator[](int i) const { return v_[i]; }

 private:
  std::size_t v_[N];
};

// parallel_for over a 2-D range: a plain double loop on the host.
class handler {
 public:
  template <typename Kernel>
  void parallel_for(range<2> r, const Kernel& k) {
    for (std::size_t i = 0; i < r[0]; ++i)
      for (std::size_t j = 0; j < r[1]; ++j) k(id<2>(i, j));
  }
};

class queue {
 public:
  template <typename Fn>
  void submit(Fn&& fn) {
    handler h;
    fn(h);
  }
  void wait() {}
};

}  // namespace sycl
