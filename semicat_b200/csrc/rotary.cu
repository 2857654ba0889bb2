// Rotary position embedding fused with the cast to the attention kernels' 16-bit input type.
//
// The denoiser rotates q and k in fp32 (semicat/net/duo.py:52-53, non-interleaved halves) and safe_sdpa_jvp then
// casts them to bf16 (semicat/jvp_utils/functional.py:318-321); under forward-mode AD every one of those
// pointwise steps runs once for the primal and once for the tangent.  This kernel does rotation and rounding in
// one pass over a strided (B, S, H, D) view and writes a contiguous (B, S, H, D) tensor:
//   y[..., :D/2] = x1 * cos - x2 * sin        y[..., D/2:] = x1 * sin + x2 * cos         (transpose = 0)
//   y[..., :D/2] = x1 * cos + x2 * sin        y[..., D/2:] = x2 * cos - x1 * sin         (transpose = 1: the VJP)
// Products and sums are separate fp32 roundings (no fused multiply-add), so the result equals the fp32 PyTorch
// formula rounded once to the output type, bit for bit.  The map is linear: the same kernel serves the tangent.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "jvpattn_common.cuh"

namespace jvpattn {
namespace {

template <typename T> struct Io;
template <> struct Io<float> {
  static __device__ __forceinline__ float load(const float *p) { return *p; }
  static __device__ __forceinline__ void store(float *p, float v) { *p = v; }
};
template <> struct Io<__nv_bfloat16> {
  static __device__ __forceinline__ float load(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
};
template <> struct Io<__half> {
  static __device__ __forceinline__ float load(const __half *p) { return __half2float(*p); }
  static __device__ __forceinline__ void store(__half *p, float v) { *p = __float2half_rn(v); }
};

// 8 consecutive elements as fp32, by 16-byte accesses (pointers 16-byte aligned)
template <typename T> struct Vec8 {
  static __device__ __forceinline__ void load(const T *p, float (&f)[8]) {
    const uint4 u = *reinterpret_cast<const uint4 *>(p);
    const T *e = reinterpret_cast<const T *>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = Io<T>::load(e + i);
  }
  static __device__ __forceinline__ void store(T *p, const float (&f)[8]) {
    uint4 u;
    T *e = reinterpret_cast<T *>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) Io<T>::store(e + i, f[i]);
    *reinterpret_cast<uint4 *>(p) = u;
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float *p, float (&f)[8]) {
    const float4 a = reinterpret_cast<const float4 *>(p)[0], b = reinterpret_cast<const float4 *>(p)[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  static __device__ __forceinline__ void store(float *p, const float (&f)[8]) {
    reinterpret_cast<float4 *>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4 *>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
  }
};

// One thread = 8 consecutive channels of the first half of one (b, s, h) row and the matching 8 of the second half.
template <typename TI, typename TO, bool kVec>
__global__ void __launch_bounds__(256) rotary_cast_kernel(const TI *x, int64_t sb, int64_t ss, int64_t sh, TO *y,
                                                          const float *cosv, const float *sinv, int B, int S, int H, int D,
                                                          int transpose) {
  const int half = D / 2, per_row = half / 8;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t rows = (int64_t)B * S * H;
  const int64_t r = gid / per_row;
  if (r >= rows) return;
  const int c0 = (int)(gid % per_row) * 8;
  const int h = (int)(r % H);
  const int s = (int)((r / H) % S);
  const int b = (int)(r / ((int64_t)H * S));
  const TI *xr = x + b * sb + s * ss + h * sh;
  TO *yr = y + r * D;
  const float *cr = cosv + (int64_t)s * half + c0, *sr = sinv + (int64_t)s * half + c0;
  float x1[8], x2[8], c[8], sn[8], y1[8], y2[8];
  if (kVec) {
    Vec8<TI>::load(xr + c0, x1);
    Vec8<TI>::load(xr + half + c0, x2);
    Vec8<float>::load(cr, c);
    Vec8<float>::load(sr, sn);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      x1[i] = Io<TI>::load(xr + c0 + i);
      x2[i] = Io<TI>::load(xr + half + c0 + i);
      c[i] = cr[i];
      sn[i] = sr[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (transpose) {
      y1[i] = __fadd_rn(__fmul_rn(x1[i], c[i]), __fmul_rn(x2[i], sn[i]));
      y2[i] = __fsub_rn(__fmul_rn(x2[i], c[i]), __fmul_rn(x1[i], sn[i]));
    } else {
      y1[i] = __fsub_rn(__fmul_rn(x1[i], c[i]), __fmul_rn(x2[i], sn[i]));
      y2[i] = __fadd_rn(__fmul_rn(x1[i], sn[i]), __fmul_rn(x2[i], c[i]));
    }
  }
  if (kVec) {
    Vec8<TO>::store(yr + c0, y1);
    Vec8<TO>::store(yr + half + c0, y2);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      Io<TO>::store(yr + c0 + i, y1[i]);
      Io<TO>::store(yr + half + c0 + i, y2[i]);
    }
  }
}

template <typename TI, typename TO>
cudaError_t launch(const void *x, int64_t sb, int64_t ss, int64_t sh, void *y, const float *cosv, const float *sinv, int B,
                   int S, int H, int D, int transpose, cudaStream_t stream) {
  const int64_t threads = (int64_t)B * S * H * (D / 16);
  if (threads == 0) return cudaSuccess;
  // 16-byte accesses when every row of x, y and the tables starts on a 16-byte boundary
  const bool vec = reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(cosv) % 16 == 0 && reinterpret_cast<uintptr_t>(sinv) % 16 == 0 &&
                   sb % 8 == 0 && ss % 8 == 0 && sh % 8 == 0;
  {
    LaunchScope scope(kIdRotary, stream);
    const unsigned grid = (unsigned)((threads + 255) / 256);
    if (vec)
      rotary_cast_kernel<TI, TO, true><<<grid, 256, 0, stream>>>(static_cast<const TI *>(x), sb, ss, sh, static_cast<TO *>(y),
                                                                 cosv, sinv, B, S, H, D, transpose);
    else
      rotary_cast_kernel<TI, TO, false><<<grid, 256, 0, stream>>>(static_cast<const TI *>(x), sb, ss, sh, static_cast<TO *>(y),
                                                                  cosv, sinv, B, S, H, D, transpose);
  }
  return cudaGetLastError();
}

// ---- q, k and v of one projection in one launch.  The block splits its qkv projection (B, S, 3, H, D) into three
// (B, S, H, D) tensors, rotates two of them and hands all three to the attention; in the backward the three gradients
// have to come back as one (B, S, 3, H, D) tensor.  With one kernel over three (input view, output view) pairs - rotation
// for the first two, a plain copy for the third - the forward is one launch instead of two plus a strided read, and the
// backward writes the projection's gradient in place instead of three tensors that PyTorch then concatenates.
struct QkvArgs {
  const void *in[3];
  void *out[3];
  int64_t isb[3], iss[3], ish[3], osb[3], oss[3], osh[3];  // element strides of (batch, position, head); channels are unit
  const float *cosv, *sinv;
  int B, S, H, D, transpose;
};

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) rotary_qkv_kernel(QkvArgs a) {
  const int half = a.D / 2, per_row = half / 8;
  const int64_t rows = (int64_t)a.B * a.S * a.H;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t rr = gid / per_row;
  if (rr >= 3 * rows) return;
  const int t = (int)(rr / rows);
  const int64_t r = rr % rows;
  const int c0 = (int)(gid % per_row) * 8;
  const int h = (int)(r % a.H);
  const int s = (int)((r / a.H) % a.S);
  const int b = (int)(r / ((int64_t)a.H * a.S));
  const TI *xr = static_cast<const TI *>(a.in[t]) + b * a.isb[t] + s * a.iss[t] + h * a.ish[t];
  TO *yr = static_cast<TO *>(a.out[t]) + b * a.osb[t] + s * a.oss[t] + h * a.osh[t];
  float x1[8], x2[8], y1[8], y2[8];
  Vec8<TI>::load(xr + c0, x1);
  Vec8<TI>::load(xr + half + c0, x2);
  if (t < 2) {
    float c[8], sn[8];
    Vec8<float>::load(a.cosv + (int64_t)s * half + c0, c);
    Vec8<float>::load(a.sinv + (int64_t)s * half + c0, sn);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (a.transpose) {
        y1[i] = __fadd_rn(__fmul_rn(x1[i], c[i]), __fmul_rn(x2[i], sn[i]));
        y2[i] = __fsub_rn(__fmul_rn(x2[i], c[i]), __fmul_rn(x1[i], sn[i]));
      } else {
        y1[i] = __fsub_rn(__fmul_rn(x1[i], c[i]), __fmul_rn(x2[i], sn[i]));
        y2[i] = __fadd_rn(__fmul_rn(x1[i], sn[i]), __fmul_rn(x2[i], c[i]));
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) y1[i] = x1[i], y2[i] = x2[i];
  }
  Vec8<TO>::store(yr + c0, y1);
  Vec8<TO>::store(yr + half + c0, y2);
}

template <typename TI, typename TO>
cudaError_t launch_qkv(const QkvArgs &a, cudaStream_t stream) {
  const int64_t threads = (int64_t)3 * a.B * a.S * a.H * (a.D / 16);
  if (threads == 0) return cudaSuccess;
  LaunchScope scope(kIdRotary, stream);
  rotary_qkv_kernel<TI, TO><<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace

// dtype codes: 0 bf16, 1 fp16, 2 fp32 (include/jvpattn.h)
cudaError_t rotary_cast(const void *x, int64_t sb, int64_t ss, int64_t sh, int in_dtype, void *y, int out_dtype,
                        const float *cosv, const float *sinv, int B, int S, int H, int D, int transpose, cudaStream_t stream) {
#define JVP_ROT(TI, TO) return launch<TI, TO>(x, sb, ss, sh, y, cosv, sinv, B, S, H, D, transpose, stream)
  switch (in_dtype * 3 + out_dtype) {
    case 0: JVP_ROT(__nv_bfloat16, __nv_bfloat16);
    case 1: JVP_ROT(__nv_bfloat16, __half);
    case 2: JVP_ROT(__nv_bfloat16, float);
    case 3: JVP_ROT(__half, __nv_bfloat16);
    case 4: JVP_ROT(__half, __half);
    case 5: JVP_ROT(__half, float);
    case 6: JVP_ROT(float, __nv_bfloat16);
    case 7: JVP_ROT(float, __half);
    case 8: JVP_ROT(float, float);
    default: return cudaErrorInvalidValue;
  }
#undef JVP_ROT
}

cudaError_t rotary_qkv(const void *const in[3], const int64_t in_strides[9], int in_dtype, void *const out[3],
                       const int64_t out_strides[9], int out_dtype, const float *cosv, const float *sinv, int B, int S, int H, int D,
                       int transpose, cudaStream_t stream) {
  QkvArgs a{};
  for (int t = 0; t < 3; ++t) {
    a.in[t] = in[t];
    a.out[t] = out[t];
    a.isb[t] = in_strides[3 * t], a.iss[t] = in_strides[3 * t + 1], a.ish[t] = in_strides[3 * t + 2];
    a.osb[t] = out_strides[3 * t], a.oss[t] = out_strides[3 * t + 1], a.osh[t] = out_strides[3 * t + 2];
  }
  a.cosv = cosv, a.sinv = sinv, a.B = B, a.S = S, a.H = H, a.D = D, a.transpose = transpose;
#define JVP_QKV(TI, TO) return launch_qkv<TI, TO>(a, stream)
  switch (in_dtype * 3 + out_dtype) {
    case 0: JVP_QKV(__nv_bfloat16, __nv_bfloat16);
    case 2: JVP_QKV(__nv_bfloat16, float);
    case 6: JVP_QKV(float, __nv_bfloat16);
    case 8: JVP_QKV(float, float);
    default: return cudaErrorInvalidValue;
  }
#undef JVP_QKV
}

}  // namespace jvpattn
