// Vocabulary-side ends of the flow-map training step, each as one pass family over (rows, V) with nothing of that
// size materialised in fp32 (semicat/models/semicat.py:70-85 interpolation, :89-110 cross-entropy step, :112-167
// self-distillation step with sd_type "lag", :210-229 flow map):
//
//   interp       xt   = (1 - t) x0 + t onehot(id)                            -> 16-bit, row pitch padded for the embedding GEMM
//   xst          xst  = xs + dt (softmax(l) - xs),  xs = (1 - s) x0 + s onehot(id),  dt = (t - s) / (1 - s + 1e-8)
//                                                                             -> 16-bit padded (input of the target pass); lse
//   ce_fwd/bwd   cross-entropy of padded 16-bit logits against ids (label smoothing eps), per-row loss and d loss / d logits
//   sd_fwd/bwd   sum_v ((1 - t) dv - softmax(l_target) + xst)^2 per row, with
//                dv = ddt (p - xs) + dt p o (tl - sum(p tl)),  ddt = 1 / (1 - s + 1e-8)   (the t-derivative of the flow map
//                by forward mode: l are the logits, tl their tangent), and its gradient with respect to l and tl.
//
// x0 is the fp32 noise (row pitch ldx), everything else is recomputed per element, so the only (rows, V) traffic is the
// operands themselves.  One CTA per (b, l) row; rows are walked in chunks of 8 columns with 16-byte accesses; columns at
// or beyond V (the padding of the GEMM operands) read as -inf logits / zero inputs and are written as zeros.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "jvpattn_common.cuh"

namespace jvpattn {
namespace {

constexpr int kThreads = 256;
constexpr float kNegInf = -INFINITY;

template <typename T> struct Pack8;
template <> struct Pack8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4 *>(p);
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16 *p, const float (&v)[8]) {
    uint4 u;
    __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4 *>(p) = u;
  }
};
template <> struct Pack8<float> {
  static __device__ __forceinline__ void load(const float *p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float *p, const float (&v)[8]) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4 *>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};

// fp32 noise row: 16-byte loads where the pitch allows (kVec), element loads with a bound otherwise
template <bool kVec>
__device__ __forceinline__ void load_x0(const float *row, int v0, int V, float (&x)[8]) {
  if (kVec) {
    Pack8<float>::load(row + v0, x);  // the padded pitch covers the whole chunk
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = v0 + i < V ? row[v0 + i] : 0.f;
  }
}

template <int NQ>
__device__ __forceinline__ void block_sum(float (&v)[NQ], float *scratch) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int q = 0; q < NQ; ++q)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v[q] += __shfl_xor_sync(0xffffffffu, v[q], o);
  __syncthreads();  // scratch may still be read from an earlier reduction
  if (lane == 0)
#pragma unroll
    for (int q = 0; q < NQ; ++q) scratch[q * 8 + warp] = v[q];
  __syncthreads();
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    float r = scratch[q * 8];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) r += scratch[q * 8 + w];
    v[q] = r;
  }
}

// Running (max, sum of exp) of one thread's elements, then across the block: returns the row's log-sum-exp.
struct OnlineLse {
  float mx = kNegInf, sm = 0.f;
  __device__ __forceinline__ void add8(const float (&l)[8]) {
    float cm = l[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) cm = fmaxf(cm, l[i]);
    if (cm == kNegInf) return;
    if (cm > mx) {
      sm *= __expf(mx - cm);  // exp(-inf) = 0 on the first chunk
      mx = cm;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sm += __expf(l[i] - mx);
  }
  __device__ __forceinline__ float finish(float *scratch) {
    float m = mx;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = m;
    __syncthreads();
    float M = scratch[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) M = fmaxf(M, scratch[w]);
    float s[1] = {mx == kNegInf ? 0.f : sm * __expf(mx - M)};
    block_sum<1>(s, scratch);
    return M + __logf(s[0]);
  }
};

template <typename T>
__device__ __forceinline__ void load_logits(const T *row, int v0, int V, float (&l)[8]) {
  Pack8<T>::load(row + v0, l);
  if (v0 + 8 > V) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (v0 + i >= V) l[i] = kNegInf;
  }
}

struct VocabArgs {
  const void *l, *tl, *lt;     // logits, their tangent, target logits: 16-bit or fp32, row pitch ld (elements, multiple of 8)
  int64_t ld;
  const float *x0;             // noise, row pitch ldx
  int64_t ldx;
  const int64_t *ids;          // [rows]
  const float *s, *t;          // [batch]
  float *lse;                  // [rows]
  float *stats;                // [rows, 4]: lse of the target logits, m = sum(p tl), sum(p r), sum(p r tl)
  float *loss;                 // [rows]
  const float *g;              // scalar cotangent of the MEAN of the row losses (device memory)
  void *out, *out2;            // 16-bit / fp32 outputs, row pitch ldo
  int64_t ldo;
  float eps;                   // label smoothing
  int rows_per_sample, V;
  int64_t rows;
};

// ------------------------------------------------------------------------------------------------ interpolation
template <typename T, bool kVec>
__global__ void __launch_bounds__(kThreads) interp_kernel(VocabArgs a) {
  const int64_t row = blockIdx.x;
  const float t = a.t[row / a.rows_per_sample];
  const int id = (int)a.ids[row];
  const float *x0 = a.x0 + row * a.ldx;
  T *out = static_cast<T *>(a.out) + row * a.ldo;
  const int nchunk = (int)(a.ldo / 8);
  for (int c = threadIdx.x; c < nchunk; c += kThreads) {
    const int v0 = c * 8;
    float x[8];
    if (v0 < a.V) {
      load_x0<kVec>(x0, v0, a.V, x);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = v0 + i < a.V ? (1.f - t) * x[i] + (v0 + i == id ? t : 0.f) : 0.f;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = 0.f;
    }
    Pack8<T>::store(out + v0, x);
  }
}

// ------------------------------------------------------------------------------------------------ flow map, primal
template <typename T, bool kVec>
__global__ void __launch_bounds__(kThreads) xst_kernel(VocabArgs a) {
  __shared__ float scratch[8];
  const int64_t row = blockIdx.x;
  const int b = (int)(row / a.rows_per_sample);
  const float s = a.s[b], t = a.t[b], dt = (t - s) / (1.f - s + 1e-8f);
  const int id = (int)a.ids[row], V = a.V;
  const T *l = static_cast<const T *>(a.l) + row * a.ld;
  const float *x0 = a.x0 + row * a.ldx;
  T *out = static_cast<T *>(a.out) + row * a.ldo;
  const int nchunk = (V + 7) / 8;
  OnlineLse acc;
  for (int c = threadIdx.x; c < nchunk; c += kThreads) {
    float lv[8];
    load_logits<T>(l, c * 8, V, lv);
    acc.add8(lv);
  }
  const float lse = acc.finish(scratch);
  if (threadIdx.x == 0) a.lse[row] = lse;
  const int nout = (int)(a.ldo / 8);
  for (int c = threadIdx.x; c < nout; c += kThreads) {
    const int v0 = c * 8;
    float o[8];
    if (c < nchunk) {
      float lv[8], x[8];
      load_logits<T>(l, v0, V, lv);
      load_x0<kVec>(x0, v0, V, x);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xs = (1.f - s) * x[i] + (v0 + i == id ? s : 0.f);
        o[i] = v0 + i < V ? xs + dt * (__expf(lv[i] - lse) - xs) : 0.f;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = 0.f;
    }
    Pack8<T>::store(out + v0, o);
  }
}

// ------------------------------------------------------------------------------------------------ cross-entropy
template <typename T>
__global__ void __launch_bounds__(kThreads) ce_fwd_kernel(VocabArgs a) {
  __shared__ float scratch[16];
  const int64_t row = blockIdx.x;
  const int id = (int)a.ids[row], V = a.V;
  const T *l = static_cast<const T *>(a.l) + row * a.ld;
  const int nchunk = (V + 7) / 8;
  OnlineLse acc;
  float sums[2] = {0.f, 0.f};  // sum of the logits (label smoothing), the target's logit
  for (int c = threadIdx.x; c < nchunk; c += kThreads) {
    float lv[8];
    load_logits<T>(l, c * 8, V, lv);
    acc.add8(lv);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (c * 8 + i < V) sums[0] += lv[i];
      if (c * 8 + i == id) sums[1] = lv[i];
    }
  }
  const float lse = acc.finish(scratch);
  block_sum<2>(sums, scratch);
  if (threadIdx.x == 0) {
    a.lse[row] = lse;
    a.loss[row] = (1.f - a.eps) * (lse - sums[1]) + a.eps * (lse - sums[0] / (float)V);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) ce_bwd_kernel(VocabArgs a) {
  const int64_t row = blockIdx.x;
  const int id = (int)a.ids[row], V = a.V;
  const T *l = static_cast<const T *>(a.l) + row * a.ld;
  T *dl = static_cast<T *>(a.out) + row * a.ldo;
  const float lse = a.lse[row], gs = a.g[0] / (float)a.rows, off = a.eps / (float)V;
  const int nchunk = (V + 7) / 8, nout = (int)(a.ldo / 8);
  for (int c = threadIdx.x; c < nout; c += kThreads) {
    const int v0 = c * 8;
    float o[8];
    if (c < nchunk) {
      float lv[8];
      load_logits<T>(l, v0, V, lv);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        o[i] = v0 + i < V ? gs * (__expf(lv[i] - lse) - (v0 + i == id ? 1.f - a.eps : 0.f) - off) : 0.f;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = 0.f;
    }
    Pack8<T>::store(dl + v0, o);
  }
}

// ------------------------------------------------------------------------------------------------ self-distillation ("lag")
// The residual of one element; shared by the forward and the backward so that both see the same value.
struct SdRow {
  float s, t, dt, ddt, lse, lse_t, m;
  int id;
  __device__ __forceinline__ float residual(float l, float tl, float lt, float x0, int v, float &p) const {
    p = __expf(l - lse);
    const float xs = (1.f - s) * x0 + (v == id ? s : 0.f);
    const float xst = xs + dt * (p - xs);
    const float dv = ddt * (p - xs) + dt * p * (tl - m);
    return (1.f - t) * dv - __expf(lt - lse_t) + xst;
  }
};

template <typename T, bool kVec>
__global__ void __launch_bounds__(kThreads) sd_fwd_kernel(VocabArgs a) {
  __shared__ float scratch[24];
  const int64_t row = blockIdx.x;
  const int b = (int)(row / a.rows_per_sample), V = a.V;
  SdRow r;
  r.s = a.s[b], r.t = a.t[b];
  r.ddt = 1.f / (1.f - r.s + 1e-8f);
  r.dt = (r.t - r.s) * r.ddt;
  r.id = (int)a.ids[row];
  r.lse = a.lse[row];
  const T *l = static_cast<const T *>(a.l) + row * a.ld;
  const T *tl = static_cast<const T *>(a.tl) + row * a.ld;
  const T *lt = static_cast<const T *>(a.lt) + row * a.ld;
  const float *x0 = a.x0 + row * a.ldx;
  const int nchunk = (V + 7) / 8;
  OnlineLse acc;
  float m[1] = {0.f};
  for (int c = threadIdx.x; c < nchunk; c += kThreads) {
    float lv[8], tv[8], qv[8];
    load_logits<T>(l, c * 8, V, lv);
    Pack8<T>::load(tl + c * 8, tv);
    load_logits<T>(lt, c * 8, V, qv);
    acc.add8(qv);
#pragma unroll
    for (int i = 0; i < 8; ++i) m[0] += __expf(lv[i] - r.lse) * (c * 8 + i < V ? tv[i] : 0.f);
  }
  r.lse_t = acc.finish(scratch);
  block_sum<1>(m, scratch);
  r.m = m[0];
  float sums[3] = {0.f, 0.f, 0.f};  // sum r^2, sum p r, sum p r tl
  for (int c = threadIdx.x; c < nchunk; c += kThreads) {
    const int v0 = c * 8;
    float lv[8], tv[8], qv[8], x[8];
    load_logits<T>(l, v0, V, lv);
    Pack8<T>::load(tl + v0, tv);
    load_logits<T>(lt, v0, V, qv);
    load_x0<kVec>(x0, v0, V, x);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (v0 + i >= V) continue;
      float p;
      const float res = r.residual(lv[i], tv[i], qv[i], x[i], v0 + i, p);
      sums[0] += res * res;
      sums[1] += p * res;
      sums[2] += p * res * tv[i];
    }
  }
  block_sum<3>(sums, scratch);
  if (threadIdx.x == 0) {
    a.loss[row] = sums[0];
    float4 st = make_float4(r.lse_t, r.m, sums[1], sums[2]);
    *reinterpret_cast<float4 *>(a.stats + row * 4) = st;
  }
}

template <typename T, bool kVec>
__global__ void __launch_bounds__(kThreads) sd_bwd_kernel(VocabArgs a) {
  const int64_t row = blockIdx.x;
  const int b = (int)(row / a.rows_per_sample), V = a.V;
  SdRow r;
  r.s = a.s[b], r.t = a.t[b];
  r.ddt = 1.f / (1.f - r.s + 1e-8f);
  r.dt = (r.t - r.s) * r.ddt;
  r.id = (int)a.ids[row];
  r.lse = a.lse[row];
  const float4 st = *reinterpret_cast<const float4 *>(a.stats + row * 4);
  r.lse_t = st.x, r.m = st.y;
  // cotangent on dv: H = gamma * residual, gamma = 2 (1 - t) g / rows; its row sums follow from the forward's
  const float gamma = 2.f * (1.f - r.t) * a.g[0] / (float)a.rows;
  const float sH = gamma * st.z, sHt = gamma * st.w;
  const float spc = r.ddt * sH + r.dt * sHt - 2.f * r.dt * r.m * sH;
  const T *l = static_cast<const T *>(a.l) + row * a.ld;
  const T *tl = static_cast<const T *>(a.tl) + row * a.ld;
  const T *lt = static_cast<const T *>(a.lt) + row * a.ld;
  const float *x0 = a.x0 + row * a.ldx;
  T *dl = static_cast<T *>(a.out) + row * a.ldo;
  T *dtl = static_cast<T *>(a.out2) + row * a.ldo;
  const int nchunk = (V + 7) / 8, nout = (int)(a.ldo / 8);
  for (int c = threadIdx.x; c < nout; c += kThreads) {
    const int v0 = c * 8;
    float o1[8], o2[8];
    if (c < nchunk) {
      float lv[8], tv[8], qv[8], x[8];
      load_logits<T>(l, v0, V, lv);
      Pack8<T>::load(tl + v0, tv);
      load_logits<T>(lt, v0, V, qv);
      load_x0<kVec>(x0, v0, V, x);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (v0 + i >= V) {
          o1[i] = o2[i] = 0.f;
          continue;
        }
        float p;
        const float H = gamma * r.residual(lv[i], tv[i], qv[i], x[i], v0 + i, p);
        const float cc = r.ddt * H + r.dt * H * (tv[i] - r.m) - r.dt * sH * tv[i];
        o1[i] = p * (cc - spc);
        o2[i] = r.dt * p * (H - sH);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) o1[i] = o2[i] = 0.f;
    }
    Pack8<T>::store(dl + v0, o1);
    Pack8<T>::store(dtl + v0, o2);
  }
}

bool aligned16(const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

}  // namespace

// op: 0 interp, 1 xst, 2 ce forward, 3 ce backward, 4 sd forward, 5 sd backward
cudaError_t vocab_loss(int op, const void *l, const void *tl, const void *lt, int64_t ld, const float *x0, int64_t ldx,
                       const int64_t *ids, const float *s, const float *t, float *lse, float *stats, float *loss, const float *g,
                       void *out, void *out2, int64_t ldo, float eps, int batch, int rows_per_sample, int V, int dtype,
                       cudaStream_t stream) {
  const int64_t rows = (int64_t)batch * rows_per_sample;
  if (rows == 0) return cudaSuccess;
  if (rows > 0x7fffffffLL) return cudaErrorInvalidValue;
  const int64_t Vp = (V + 7) & ~7;
  // 16-byte accesses: every 16-bit / fp32 operand row must start on a 16-byte boundary and cover the padded width
  for (const void *p : {l, tl, lt})
    if (p && (!aligned16(p) || ld % 8 || ld < Vp)) return cudaErrorInvalidValue;
  for (const void *p : {(const void *)out, (const void *)out2})
    if (p && (!aligned16(p) || ldo % 8 || ldo < Vp)) return cudaErrorInvalidValue;
  if (stats && !aligned16(stats)) return cudaErrorInvalidValue;
  const bool vec = x0 && aligned16(x0) && ldx % 4 == 0 && ldx >= Vp;
  VocabArgs a{l, tl, lt, ld, x0, ldx, ids, s, t, lse, stats, loss, g, out, out2, ldo, eps, rows_per_sample, V, rows};
  LaunchScope scope(kIdDual, stream);
  auto launch = [&](auto tag) -> cudaError_t {
    using T = decltype(tag);
    const dim3 grid((unsigned)rows), block(kThreads);
    switch (op) {
      case 0: vec ? interp_kernel<T, true><<<grid, block, 0, stream>>>(a) : interp_kernel<T, false><<<grid, block, 0, stream>>>(a); break;
      case 1: vec ? xst_kernel<T, true><<<grid, block, 0, stream>>>(a) : xst_kernel<T, false><<<grid, block, 0, stream>>>(a); break;
      case 2: ce_fwd_kernel<T><<<grid, block, 0, stream>>>(a); break;
      case 3: ce_bwd_kernel<T><<<grid, block, 0, stream>>>(a); break;
      case 4: vec ? sd_fwd_kernel<T, true><<<grid, block, 0, stream>>>(a) : sd_fwd_kernel<T, false><<<grid, block, 0, stream>>>(a); break;
      case 5: vec ? sd_bwd_kernel<T, true><<<grid, block, 0, stream>>>(a) : sd_bwd_kernel<T, false><<<grid, block, 0, stream>>>(a); break;
      default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
  };
  if (dtype == JVPATTN_BF16) return launch(__nv_bfloat16{});
  if (dtype == JVPATTN_FP32) return launch(float{});
  return cudaErrorInvalidValue;
}

}  // namespace jvpattn
