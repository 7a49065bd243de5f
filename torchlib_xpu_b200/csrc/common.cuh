// Shared device helpers for the b200tbe kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "b200tbe.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "b200tbe is written for sm_100a (B200) only"
#endif

namespace b200tbe {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this
constexpr int kWarpSize = 32;
constexpr unsigned kFullMask = 0xffffffffu;

inline int launch_status() {
  return cudaGetLastError() == cudaSuccess ? B200TBE_OK : B200TBE_ERR_LAUNCH;
}

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// 16-byte read-only load that does not allocate in L1: embedding rows and streamed copies have no
// reuse inside one SM, while L2 (126 MB) is where repeated rows are meant to hit.
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t ldg_stream4(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// Streaming 16-byte store (evict-first): outputs are written once and not re-read by the kernel.
__device__ __forceinline__ void stg_stream16(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

__device__ __forceinline__ void stg_stream8(void* p, uint2 v) {
  asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

template <typename IndexT>
__device__ __forceinline__ int64_t load_index(const void* base, int64_t i) {
  return static_cast<int64_t>(__ldg(reinterpret_cast<const IndexT*>(base) + i));
}

__device__ __forceinline__ float2 half2_bits_to_float2(uint32_t h2) {
  return __half22float2(*reinterpret_cast<const __half2*>(&h2));
}

__device__ __forceinline__ uint32_t float2_to_half2_bits(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
  return v;
}

}  // namespace b200tbe
