// Small device/host helpers shared by the tcgen05 attention kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "jvpattn_common.cuh"

namespace jvpattn {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}

template <typename T> struct IsBf16 { static constexpr bool value = false; };
template <> struct IsBf16<__nv_bfloat16> { static constexpr bool value = true; };

// A view the TMA / vector-store paths can take: 16-byte aligned base, strides that keep every row 16-byte
// aligned, rows that do not overlap.
inline bool tma_view_ok(const View &v, int D) {
  if (!v.ptr) return false;
  if (reinterpret_cast<uintptr_t>(v.ptr) % 16 != 0) return false;
  return v.sl % 8 == 0 && v.sh % 8 == 0 && v.sb % 8 == 0 && v.sl >= D;
}

}  // namespace jvpattn
