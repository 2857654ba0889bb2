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
// aligned, rows that do not overlap, and a positive stride below 2^40 bytes on every axis that has more than one
// entry (a tensor map cannot describe a broadcast axis; an expanded tensor takes the SIMT kernels instead).
inline bool tma_view_ok(const View &v, int B, int H, int L, int D) {
  if (!v.ptr) return false;
  if (reinterpret_cast<uintptr_t>(v.ptr) % 16 != 0) return false;
  auto axis_ok = [](int64_t stride, int n) { return n <= 1 || (stride > 0 && stride % 8 == 0 && stride < (int64_t(1) << 39)); };
  return axis_ok(v.sl, L) && axis_ok(v.sh, H) && axis_ok(v.sb, B) && (L <= 1 || v.sl >= D);
}

}  // namespace jvpattn
