// Vocabulary-side head of the flow-map step on (primal, tangent) pairs:
//   xst = x + dt (softmax(l) - x)                              (semicat/models/semicat.py:210-229, the flow map)
//   dv  = ddt (p - x) + dt p o (tl - sum(p tl))                 (its derivative in t by forward mode, semicat.py:153-157)
// with l the denoiser's logits over the vocabulary (B, L, V), tl their tangent, x the interpolated input (fp32, no
// tangent), dt = (t - s) / (1 - s) per sample and ddt its derivative.  PyTorch runs this as a softmax, its tangent and
// half a dozen pointwise passes over (B, L, V) fp32 tensors (tens of GB per step at V = 30522), and as many again in
// the backward.  One CTA owns one (b, l) row: the logits (and their tangent) are staged once in shared memory in their
// 16-bit or fp32 storage type, row sums are block reductions, every global tensor is read or written once per kernel.
//
// VJPs (cotangents G on xst, H on dv; softmax Jacobians are symmetric):
//   G:  dl  = dt p o (G - sum(p G))
//   H:  dtl = dt p o (H - sum(p H))
//       dl  = p o (c - sum(p c)),   c = ddt H + dt H o (tl - m) - dt sum(p H) tl,   m = sum(p tl)
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "jvpattn_common.cuh"

namespace jvpattn {
namespace {

constexpr int kThreads = 512;

template <typename T> __device__ __forceinline__ float ldf(const T *p);
template <> __device__ __forceinline__ float ldf<float>(const float *p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T *p, float v);
template <> __device__ __forceinline__ void stf<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

// Block-wide sum (or max) of up to NQ values per thread; every thread gets the results.
template <int NQ, bool kMax>
__device__ __forceinline__ void block_reduce(float (&v)[NQ], float *scratch) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int q = 0; q < NQ; ++q)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, v[q], o);
      v[q] = kMax ? fmaxf(v[q], other) : v[q] + other;
    }
  __syncthreads();  // scratch may still be read from an earlier reduction
  if (lane == 0)
#pragma unroll
    for (int q = 0; q < NQ; ++q) scratch[q * 16 + warp] = v[q];
  __syncthreads();
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    float r = scratch[q * 16];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) r = kMax ? fmaxf(r, scratch[q * 16 + w]) : r + scratch[q * 16 + w];
    v[q] = r;
  }
}

struct HeadArgs {
  const void *l, *tl;        // logits and their tangent: rows `ldl` / `ldt` elements apart
  int64_t ldl, ldt;
  const float *x;            // [rows, V] contiguous
  const float *dt, *ddt;     // [B]
  float *lse;                // [rows]: log-sum-exp of the logits (written by the forward, read by the others)
  float *out;                // forward: xst or dv, [rows, V]
  const float *g;            // cotangent [rows, V]
  void *dl, *dtl;            // gradients, contiguous [rows, V] in the logits' type
  int rows_per_sample, V;
};

// which: 0 forward (xst, lse), 1 forward tangent (dv), 2 VJP of xst, 3 VJP of dv
template <typename T, int kWhich>
__global__ void __launch_bounds__(kThreads) vocab_head_kernel(HeadArgs a) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ float scratch[4 * 16];
  T *sl = reinterpret_cast<T *>(smem_raw);
  T *stl = sl + ((a.V + 7) & ~7);
  const int64_t row = blockIdx.x;
  const int b = (int)(row / a.rows_per_sample);
  const int V = a.V;
  const T *l = static_cast<const T *>(a.l) + row * a.ldl;
  constexpr bool kNeedT = kWhich == 1 || kWhich == 3;
  const T *tl = kNeedT ? static_cast<const T *>(a.tl) + row * a.ldt : nullptr;
  // stage the row(s): 16-byte copies where the row start is 16-byte aligned (a padded projection output is), element
  // copies for the ragged tail and for unaligned rows
  {
    constexpr int kPer = 16 / (int)sizeof(T);
    const bool al = (reinterpret_cast<uintptr_t>(l) % 16 == 0) && (!kNeedT || reinterpret_cast<uintptr_t>(tl) % 16 == 0);
    const int nvec = al ? V / kPer : 0;
    for (int i = threadIdx.x; i < nvec; i += kThreads) {
      reinterpret_cast<uint4 *>(sl)[i] = reinterpret_cast<const uint4 *>(l)[i];
      if (kNeedT) reinterpret_cast<uint4 *>(stl)[i] = reinterpret_cast<const uint4 *>(tl)[i];
    }
    for (int i = nvec * kPer + threadIdx.x; i < V; i += kThreads) {
      sl[i] = l[i];
      if (kNeedT) stl[i] = tl[i];
    }
  }
  __syncthreads();
  const float dt = a.dt[b];
  float lse;
  if (kWhich == 0) {
    float m[1] = {-INFINITY};
    for (int i = threadIdx.x; i < V; i += kThreads) m[0] = fmaxf(m[0], ldf<T>(sl + i));
    block_reduce<1, true>(m, scratch);
    float s[1] = {0.f};
    for (int i = threadIdx.x; i < V; i += kThreads) s[0] += __expf(ldf<T>(sl + i) - m[0]);
    block_reduce<1, false>(s, scratch);
    lse = m[0] + __logf(s[0]);
    if (threadIdx.x == 0) a.lse[row] = lse;
  } else {
    lse = a.lse[row];
  }
  const float *x = a.x ? a.x + row * (int64_t)V : nullptr;
  if (kWhich == 0) {
    float *out = a.out + row * (int64_t)V;
    for (int i = threadIdx.x; i < V; i += kThreads) {
      const float p = __expf(ldf<T>(sl + i) - lse), xv = x[i];
      out[i] = xv + dt * (p - xv);
    }
  } else if (kWhich == 1) {
    const float ddt = a.ddt[b];
    float m[1] = {0.f};
    for (int i = threadIdx.x; i < V; i += kThreads) m[0] += __expf(ldf<T>(sl + i) - lse) * ldf<T>(stl + i);
    block_reduce<1, false>(m, scratch);
    float *out = a.out + row * (int64_t)V;
    for (int i = threadIdx.x; i < V; i += kThreads) {
      const float p = __expf(ldf<T>(sl + i) - lse);
      out[i] = ddt * (p - x[i]) + dt * p * (ldf<T>(stl + i) - m[0]);
    }
  } else if (kWhich == 2) {
    const float *g = a.g + row * (int64_t)V;
    float s[1] = {0.f};
    for (int i = threadIdx.x; i < V; i += kThreads) s[0] += __expf(ldf<T>(sl + i) - lse) * g[i];
    block_reduce<1, false>(s, scratch);
    T *dl = static_cast<T *>(a.dl) + row * (int64_t)V;
    for (int i = threadIdx.x; i < V; i += kThreads) stf<T>(dl + i, dt * __expf(ldf<T>(sl + i) - lse) * (g[i] - s[0]));
  } else {
    const float ddt = a.ddt[b];
    const float *h = a.g + row * (int64_t)V;
    float s[3] = {0.f, 0.f, 0.f};  // m = sum p tl, sH = sum p H, sHt = sum p H tl
    for (int i = threadIdx.x; i < V; i += kThreads) {
      const float p = __expf(ldf<T>(sl + i) - lse), t = ldf<T>(stl + i), hv = h[i];
      s[0] += p * t;
      s[1] += p * hv;
      s[2] += p * hv * t;
    }
    block_reduce<3, false>(s, scratch);
    const float m = s[0], sH = s[1], sHt = s[2];
    const float spc = ddt * sH + dt * sHt - 2.f * dt * m * sH;  // sum(p c)
    T *dl = static_cast<T *>(a.dl) + row * (int64_t)V;
    T *dtl = static_cast<T *>(a.dtl) + row * (int64_t)V;
    for (int i = threadIdx.x; i < V; i += kThreads) {
      const float p = __expf(ldf<T>(sl + i) - lse), t = ldf<T>(stl + i), hv = h[i];
      const float c = ddt * hv + dt * hv * (t - m) - dt * sH * t;
      stf<T>(dl + i, p * (c - spc));
      stf<T>(dtl + i, dt * p * (hv - sH));
    }
  }
}

}  // namespace

cudaError_t vocab_head(int which, const void *l, const void *tl, int64_t ldl, int64_t ldt, const float *x, const float *dt,
                       const float *ddt, float *lse, float *out, const float *g, void *dl, void *dtl, int batch,
                       int rows_per_sample, int V, int dtype, cudaStream_t stream) {
  HeadArgs a{l, tl, ldl, ldt, x, dt, ddt, lse, out, g, dl, dtl, rows_per_sample, V};
  const int64_t rows = (int64_t)batch * rows_per_sample;
  if (rows == 0) return cudaSuccess;
  const size_t esz = dtype == JVPATTN_BF16 ? 2 : 4;
  const size_t smem = ((which == 1 || which == 3) ? 2 : 1) * (size_t)((V + 7) & ~7) * esz;  // logits (+ their tangent)
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  LaunchScope scope(kIdDual, stream);
  auto launch = [&](auto t) -> cudaError_t {
    using T = decltype(t);
    auto go = [&](auto kernel) {
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      kernel<<<(unsigned)rows, kThreads, smem, stream>>>(a);
      return cudaGetLastError();
    };
    switch (which) {
      case 0: return go(vocab_head_kernel<T, 0>);
      case 1: return go(vocab_head_kernel<T, 1>);
      case 2: return go(vocab_head_kernel<T, 2>);
      case 3: return go(vocab_head_kernel<T, 3>);
      default: return cudaErrorInvalidValue;
    }
  };
  if (dtype == JVPATTN_BF16) return launch(__nv_bfloat16{});
  if (dtype == JVPATTN_FP32) return launch(float{});
  return cudaErrorInvalidValue;
}

}  // namespace jvpattn
