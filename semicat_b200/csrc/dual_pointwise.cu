// Dual-number pointwise kernels for the denoiser block around the attention: every op takes a primal and a tangent and
// returns both in one pass, and has a hand-written VJP for the cotangents of both outputs.  Under torch.func.jvp the same
// algebra runs as a dozen small kernels per op and per pass (primal and tangent separately), which is what bounds the
// training step once the batch is sharded over several GPUs.
//
//   ln_modulate     h = LN(x) * (1 + scale) + shift        (semicat/net/duo.py:128-135, 159: LayerNorm + adaLN modulation)
//   gated_residual  z = x + m * (g * y)                    (duo.py:157, 160: dropout(branch * gate) + skip; m = dropout keep
//                                                           mask / (1 - p): a tensor, or regenerated here from a seed)
//   gelu_dual       the tanh-form GELU of the MLP          (duo.py:118-123)
//
// LayerNorm: one warp owns one row of C channels (C = 256, 512, 768 or 1024; one element type, bf16 or fp32, for every
// tensor but the fp32 LayerNorm weight and bias): 16-byte loads, fp32 arithmetic, warp-shuffle row reductions; column
// sums that feed the gradients of per-sample or per-channel parameters are accumulated per CTA (registers, then one
// shared-memory slice per warp) and added to fp32 [B, C] buffers with one atomic per column and CTA (a CTA stays inside
// one sample); ln_finalize turns them into the parameter gradients.  Gated residual and GELU: 8 elements per thread.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <type_traits>

#include "jvpattn_common.cuh"

namespace jvpattn {
namespace {

constexpr int kWarpsPerCta = 4;

template <typename T>
__device__ __forceinline__ void load8(const T *p, float (&f)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float *p, float (&f)[8]) {
  const float4 a = reinterpret_cast<const float4 *>(p)[0], b = reinterpret_cast<const float4 *>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16 *p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4 *>(p);
  const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
template <typename T> __device__ __forceinline__ float ldf(const T *p);
template <> __device__ __forceinline__ float ldf<float>(const float *p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T *p, float v);
template <> __device__ __forceinline__ void stf<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
template <typename T>
__device__ __forceinline__ void store8(T *p, const float (&f)[8]);
template <>
__device__ __forceinline__ void store8<float>(float *p, const float (&f)[8]) {
  reinterpret_cast<float4 *>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
  reinterpret_cast<float4 *>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16 *p, const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4 *>(p) = u;
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// Channel index of element e of vector v of this lane: vectors of 8 channels, lanes interleaved (coalesced 16-byte loads).
__device__ __forceinline__ int chan(int v, int lane) { return (v * 32 + lane) * 8; }

struct LnArgs {
  const void *x, *tx;            // [rows, C]
  const float *gamma, *beta;     // [C] (beta may be null: no bias)
  const void *shift, *scale;     // [B, C] rows `mod_stride` elements apart
  const void *tshift, *tscale;   // tangents of shift / scale (null = zero)
  int64_t mod_stride, tmod_stride;
  float *mean, *rstd;            // [rows]
  void *y;                       // output of the forward kernels
  const void *g;                 // cotangent (backward kernels)
  void *dx, *dtx;                // gradients with respect to x / tx
  float *sums;                   // [3, B, C] fp32 column sums (zeroed by the caller)
  int B, S, C;
  float eps;
  int exact;                     // backward of the tangent: bit 0 = full second-order terms (else mean / rstd held constant),
                                 // bit 1 = add to what dx holds instead of overwriting it
};

// ---- forward.  kTangent = false: y = (n gamma + beta)(1 + scale) + shift, saves mean / rstd.
//               kTangent = true:  ty = nd gamma (1 + scale) + (n gamma + beta) tscale + tshift,  nd = rstd P_n(tx),
//               where P_n(z) = z - mean(z) - n mean(n z)
template <typename T, int NV, bool kTangent>
__global__ void __launch_bounds__(kWarpsPerCta * 32) ln_modulate_fwd_kernel(LnArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + warp;
  if (row >= (int64_t)a.B * a.S) return;
  const int b = (int)(row / a.S);
  constexpr int C = NV * 256;
  const T *x = static_cast<const T *>(a.x) + row * C;
  float xv[NV][8];
  float s = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    load8<T>(x + chan(v, lane), xv[v]);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += xv[v][i];
  }
  float mean, rstd;
  if (!kTangent) {
    mean = warp_sum(s) / C;
    float q = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d = xv[v][i] - mean;
        q += d * d;
      }
    }
    rstd = rsqrtf(warp_sum(q) / C + a.eps);
    if (lane == 0) {
      a.mean[row] = mean;
      a.rstd[row] = rstd;
    }
  } else {
    mean = a.mean[row];
    rstd = a.rstd[row];
  }
  const T *sc = static_cast<const T *>(a.scale) + (int64_t)b * a.mod_stride;
  T *y = static_cast<T *>(a.y) + row * C;
  if (!kTangent) {
    const T *sh = static_cast<const T *>(a.shift) + (int64_t)b * a.mod_stride;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c0 = chan(v, lane);
      float g[8], be[8], scv[8], shv[8], out[8];
      load8<float>(a.gamma + c0, g);
      if (a.beta) load8<float>(a.beta + c0, be);
      load8<T>(sc + c0, scv);
      load8<T>(sh + c0, shv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float ln = (xv[v][i] - mean) * rstd * g[i] + (a.beta ? be[i] : 0.f);
        out[i] = ln * (1.f + scv[i]) + shv[i];
      }
      store8<T>(y + c0, out);
    }
  } else {
    const T *tx = static_cast<const T *>(a.tx) + row * C;
    float tv[NV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      load8<T>(tx + chan(v, lane), tv[v]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        s1 += tv[v][i];
        s2 += (xv[v][i] - mean) * rstd * tv[v][i];
      }
    }
    const float m1 = warp_sum(s1) / C, m2 = warp_sum(s2) / C;
    const T *tsc = a.tscale ? static_cast<const T *>(a.tscale) + (int64_t)b * a.tmod_stride : nullptr;
    const T *tsh = a.tshift ? static_cast<const T *>(a.tshift) + (int64_t)b * a.tmod_stride : nullptr;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c0 = chan(v, lane);
      float g[8], be[8], scv[8], tscv[8], tshv[8], out[8];
      load8<float>(a.gamma + c0, g);
      if (a.beta) load8<float>(a.beta + c0, be);
      load8<T>(sc + c0, scv);
      if (tsc) load8<T>(tsc + c0, tscv);
      if (tsh) load8<T>(tsh + c0, tshv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float n = (xv[v][i] - mean) * rstd;
        const float nd = rstd * (tv[v][i] - m1 - n * m2);
        float o = nd * g[i] * (1.f + scv[i]);
        if (tsc) o += (n * g[i] + (a.beta ? be[i] : 0.f)) * tscv[i];
        if (tsh) o += tshv[i];
        out[i] = o;
      }
      store8<T>(y + c0, out);
    }
  }
}

// Column sums of a CTA: every warp parks its per-channel partial sums in its own slice of shared memory (plain stores),
// then the CTA adds the slices and issues one global atomic per column.  `smem` holds kWarpsPerCta * NQ * C floats.
template <int NQ, int NV>
__device__ __forceinline__ void flush_column_sums(float *smem, const float (&part)[NQ][NV][8], int lane, float *const (&dst)[NQ]) {
  constexpr int C = NV * 256;
  const int warp = threadIdx.x >> 5;
  float *mine = smem + (size_t)warp * NQ * C;
#pragma unroll
  for (int q = 0; q < NQ; ++q)
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      float f[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = part[q][v][i];
      store8<float>(mine + q * C + chan(v, lane), f);
    }
  __syncthreads();
  for (int q = 0; q < NQ; ++q)
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < kWarpsPerCta; ++w) t += smem[((size_t)w * NQ + q) * C + c];
      atomicAdd(dst[q] + c, t);
    }
}

// ---- backward of y.  u = G gamma (1 + scale);  dx = rstd P_n(u);  sums[0] += G n, sums[1] += G   (per sample)
template <typename T, int NV>
__global__ void __launch_bounds__(kWarpsPerCta * 32) ln_modulate_bwd_kernel(LnArgs a, int rows_per_cta) {
  extern __shared__ float smem_raw[];
  constexpr int C = NV * 256;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ctas_per_sample = (a.S + rows_per_cta - 1) / rows_per_cta;
  const int b = blockIdx.x / ctas_per_sample;
  const int s0 = (blockIdx.x % ctas_per_sample) * rows_per_cta;
  const T *sc = static_cast<const T *>(a.scale) + (int64_t)b * a.mod_stride;
  float part[2][NV][8] = {};
  for (int r = warp; r < rows_per_cta && s0 + r < a.S; r += kWarpsPerCta) {
    const int64_t row = (int64_t)b * a.S + s0 + r;
    const T *x = static_cast<const T *>(a.x) + row * C;
    const T *g = static_cast<const T *>(a.g) + row * C;
    const float mean = a.mean[row], rstd = a.rstd[row];
    float n[NV][8], u[NV][8];
    float su = 0.f, sun = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c0 = chan(v, lane);
      float xv[8], gv[8], gam[8], scv[8];
      load8<T>(x + c0, xv);
      load8<T>(g + c0, gv);
      load8<float>(a.gamma + c0, gam);
      load8<T>(sc + c0, scv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        n[v][i] = (xv[i] - mean) * rstd;
        u[v][i] = gv[i] * gam[i] * (1.f + scv[i]);
        su += u[v][i];
        sun += u[v][i] * n[v][i];
        part[0][v][i] += gv[i] * n[v][i];
        part[1][v][i] += gv[i];
      }
    }
    const float mu_ = warp_sum(su) / C, mun = warp_sum(sun) / C;
    T *dx = static_cast<T *>(a.dx) + row * C;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      float out[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] = rstd * (u[v][i] - mu_ - n[v][i] * mun);
      store8<T>(dx + chan(v, lane), out);
    }
  }
  float *const dst[2] = {a.sums + (int64_t)b * C, a.sums + ((int64_t)a.B + b) * C};
  flush_column_sums<2, NV>(smem_raw, part, lane, dst);
}

// ---- backward of ty.  u = G gamma (1 + scale), w = G gamma tscale, nd = rstd P_n(tx):
//   dtx = rstd P_n(u)
//   exact:        dx = rstd P_n(w + gn) - rstd n mean(u nd),   gn = -rstd (u mean(n tx) + tx mean(u n))
//   mean / rstd held constant inside nd (what autograd does with the forward-mode formula of native_layer_norm, whose
//   saved statistics are not differentiable outputs; the w term goes through the primal output and is differentiated
//   in full):   dx = rstd P_n(w) - rstd^2 (u mean(n tx) + (tx - mean(tx)) mean(u n))
//   sums[0] += G n, sums[1] += G, sums[2] += G nd   (per sample)
template <typename T, int NV>
__global__ void __launch_bounds__(kWarpsPerCta * 32) ln_modulate_bwd_tangent_kernel(LnArgs a, int rows_per_cta) {
  extern __shared__ float smem_raw[];
  constexpr int C = NV * 256;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ctas_per_sample = (a.S + rows_per_cta - 1) / rows_per_cta;
  const int b = blockIdx.x / ctas_per_sample;
  const int s0 = (blockIdx.x % ctas_per_sample) * rows_per_cta;
  const T *sc = static_cast<const T *>(a.scale) + (int64_t)b * a.mod_stride;
  const T *tsc = a.tscale ? static_cast<const T *>(a.tscale) + (int64_t)b * a.tmod_stride : nullptr;
  float part[3][NV][8] = {};
  for (int r = warp; r < rows_per_cta && s0 + r < a.S; r += kWarpsPerCta) {
    const int64_t row = (int64_t)b * a.S + s0 + r;
    const T *x = static_cast<const T *>(a.x) + row * C;
    const T *tx = static_cast<const T *>(a.tx) + row * C;
    const T *g = static_cast<const T *>(a.g) + row * C;
    const float mean = a.mean[row], rstd = a.rstd[row];
    float n[NV][8], t[NV][8], gv[NV][8];
    float st = 0.f, snt = 0.f, su = 0.f, sun = 0.f, sw = 0.f, swn = 0.f, sut = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c0 = chan(v, lane);
      float xv[8], gam[8], scv[8], tscv[8];
      load8<T>(x + c0, xv);
      load8<T>(tx + c0, t[v]);
      load8<T>(g + c0, gv[v]);
      load8<float>(a.gamma + c0, gam);
      load8<T>(sc + c0, scv);
      if (tsc) load8<T>(tsc + c0, tscv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        n[v][i] = (xv[i] - mean) * rstd;
        const float gg = gv[v][i] * gam[i];
        const float u = gg * (1.f + scv[i]), w = tsc ? gg * tscv[i] : 0.f;
        st += t[v][i];
        snt += n[v][i] * t[v][i];
        su += u;
        sun += u * n[v][i];
        sw += w;
        swn += w * n[v][i];
        sut += u * t[v][i];
      }
    }
    const float inv = 1.f / C;
    const float m_t = warp_sum(st) * inv, m_nt = warp_sum(snt) * inv, m_u = warp_sum(su) * inv, m_un = warp_sum(sun) * inv;
    const float m_w = warp_sum(sw) * inv, m_wn = warp_sum(swn) * inv, m_ut = warp_sum(sut) * inv;
    // nd = rstd (t - m_t - n m_nt)   =>   mean(u nd) = rstd (m_ut - m_u m_t - m_un m_nt)
    const float m_und = rstd * (m_ut - m_u * m_t - m_un * m_nt);
    // gn = -rstd (u m_nt + t m_un)   =>   mean(gn) = -rstd (m_u m_nt + m_t m_un),  mean(gn n) = -2 rstd m_un m_nt
    const float m_gn = -rstd * (m_u * m_nt + m_t * m_un), m_gnn = -2.f * rstd * m_un * m_nt;
    T *dx = static_cast<T *>(a.dx) + row * C;
    T *dtx = static_cast<T *>(a.dtx) + row * C;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int c0 = chan(v, lane);
      float gam[8], scv[8], tscv[8], o1[8], o2[8];
      load8<float>(a.gamma + c0, gam);  // (cache hits: the row loop above just read them)
      load8<T>(sc + c0, scv);
      if (tsc) load8<T>(tsc + c0, tscv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float gg = gv[v][i] * gam[i];
        const float u = gg * (1.f + scv[i]), w = tsc ? gg * tscv[i] : 0.f;
        const float nn = n[v][i], tt = t[v][i];
        const float nd = rstd * (tt - m_t - nn * m_nt);
        o2[i] = rstd * (u - m_u - nn * m_un);
        if (a.exact & 1) {
          const float gn = -rstd * (u * m_nt + tt * m_un);
          o1[i] = rstd * ((w + gn) - (m_w + m_gn) - nn * (m_wn + m_gnn)) - rstd * nn * m_und;
        } else {
          o1[i] = rstd * ((w - m_w - nn * m_wn) - rstd * (u * m_nt + (tt - m_t) * m_un));
        }
        part[0][v][i] += gv[v][i] * nn;
        part[1][v][i] += gv[v][i];
        part[2][v][i] += gv[v][i] * nd;
      }
      if (a.exact & 2) {  // dx already holds the gradient that arrived through the primal output: add to it
        float prev[8];
        load8<T>(dx + c0, prev);
#pragma unroll
        for (int i = 0; i < 8; ++i) o1[i] += prev[i];
      }
      store8<T>(dx + c0, o1);
      store8<T>(dtx + c0, o2);
    }
  }
  float *const dst[3] = {a.sums + (int64_t)b * C, a.sums + ((int64_t)a.B + b) * C, a.sums + ((int64_t)2 * a.B + b) * C};
  flush_column_sums<3, NV>(smem_raw, part, lane, dst);
}

// ---- dropout keep mask computed in the kernel instead of read from memory.  Philox-4x32-10 (Salmon et al., "Parallel
// random numbers: as easy as 1, 2, 3", 2011) keyed by a 64-bit seed that lives in device memory (drawn once per training
// step, so a replayed CUDA graph sees a new one), counter = (chunk index, call index): every kernel that touches the same
// call of the same step regenerates the same mask.  One call yields 8 x 16 bits = the masks of 8 adjacent elements.
struct DropArgs {
  const unsigned long long *seed;  // null: no generated mask
  unsigned call;
  float p;
};

__device__ __forceinline__ void dropout8(const DropArgs &d, int64_t chunk, float (&m)[8]) {
  const unsigned long long seed = *d.seed;
  unsigned k0 = (unsigned)seed, k1 = (unsigned)(seed >> 32);
  unsigned c0 = (unsigned)chunk, c1 = (unsigned)((unsigned long long)chunk >> 32), c2 = d.call, c3 = 0x5eedu;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const unsigned hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const unsigned hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0;
    c1 = lo1;
    c2 = hi0 ^ c3 ^ k1;
    c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  const float keep = 1.f - d.p, inv = 1.f / keep;
  const unsigned thr = (unsigned)(keep * 65536.f);
  const unsigned w[4] = {c0, c1, c2, c3};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[2 * i] = (w[i] & 0xffffu) < thr ? inv : 0.f;
    m[2 * i + 1] = (w[i] >> 16) < thr ? inv : 0.f;
  }
}

struct GateArgs {
  const void *x, *y;         // [rows, C]
  const void *gate;          // [B, C] rows `gate_stride` apart
  const void *mask;          // [rows, C] in the branch dtype: keep mask / (1 - p); null = all ones (or generated, see drop)
  int64_t gate_stride;
  void *z;
  int B, S, C;
  DropArgs drop;             // used when mask is null and drop.seed is not
};

// z = x + m g y without a tangent (the passes that run outside forward-mode AD)
template <typename T>
__global__ void __launch_bounds__(256) gated_residual_fwd_kernel(GateArgs a) {
  const int64_t total = (int64_t)a.B * a.S * a.C / 8;
  for (int64_t i8 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i8 < total; i8 += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = i8 * 8;
    const int c0 = (int)(e % a.C);
    const int b = (int)(e / ((int64_t)a.S * a.C));
    float xv[8], yv[8], gv[8], mv[8], out[8];
    load8<T>(static_cast<const T *>(a.x) + e, xv);
    load8<T>(static_cast<const T *>(a.y) + e, yv);
    load8<T>(static_cast<const T *>(a.gate) + (int64_t)b * a.gate_stride + c0, gv);
    const bool masked = a.mask || a.drop.seed;
    if (a.mask) load8<T>(static_cast<const T *>(a.mask) + e, mv);
    else if (a.drop.seed) dropout8(a.drop, i8, mv);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = xv[i] + (masked ? mv[i] : 1.f) * gv[i] * yv[i];
    store8<T>(static_cast<T *>(a.z) + e, out);
  }
}

// Rows of one sample that a CTA of the backward kernels walks before it adds its column sums to global memory.  Every CTA
// costs one atomic per column and sum, and at a few hundred samples those atomics (millions per launch, a dozen
// contenders per address) took longer than the rows themselves; so the count grows with the problem as long as
// eight CTAs per SM remain.
inline int rows_per_cta(int B, int S, int base) {
  int rows = base;
  while (rows < 64 && (int64_t)B * ((S + 2 * rows - 1) / (2 * rows)) >= 148 * 8) rows *= 2;
  return rows;
}

// ---- gradients of the modulation tensors and of the LayerNorm weight / bias from the column sums of the two backward
// kernels, in one launch.  p = sums of the VJP of y ([2, B, C]: sum_s g n, sum_s g), t = sums of the VJP of ty ([3, B, C]:
// sum_s g n, sum_s g, sum_s g nd); either may be null.  One thread per channel walks the samples.
struct LnFinalArgs {
  const float *p, *t;
  const float *gamma, *beta;
  const void *scale, *tscale;
  int64_t mod_stride, tmod_stride;
  void *d_shift, *d_scale, *d_tshift, *d_tscale;  // [B, C] contiguous in the modulation dtype (null = not wanted)
  float *d_gamma, *d_beta;                        // [C], zeroed by the caller: CTAs add their samples' share
  int B, C;
};

constexpr int kFinalSamples = 8;  // samples per thread of the finalize kernel

template <typename T>
__global__ void ln_finalize_kernel(LnFinalArgs a) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= a.C) return;
  const float gam = a.gamma[c], bet = a.beta ? a.beta[c] : 0.f;
  float dg = 0.f, db = 0.f;
  const int64_t BC = (int64_t)a.B * a.C;
  const int b0 = blockIdx.y * kFinalSamples, b1 = min(a.B, b0 + kFinalSamples);
#pragma unroll 4
  for (int b = b0; b < b1; ++b) {
    const int64_t i = (int64_t)b * a.C + c;
    const float sc1 = 1.f + ldf<T>(static_cast<const T *>(a.scale) + (int64_t)b * a.mod_stride + c);
    const float tsc = a.tscale ? ldf<T>(static_cast<const T *>(a.tscale) + (int64_t)b * a.tmod_stride + c) : 0.f;
    float d_scale = 0.f;
    if (a.p) {
      const float gn = a.p[i], g1 = a.p[BC + i];
      if (a.d_shift) stf<T>(static_cast<T *>(a.d_shift) + i, g1);
      d_scale += gam * gn + bet * g1;
      dg += gn * sc1;
      db += g1 * sc1;
    }
    if (a.t) {
      const float gn = a.t[i], g1 = a.t[BC + i], gnd = a.t[2 * BC + i];
      if (a.d_tshift) stf<T>(static_cast<T *>(a.d_tshift) + i, g1);
      if (a.d_tscale) stf<T>(static_cast<T *>(a.d_tscale) + i, gam * gn + bet * g1);
      d_scale += gam * gnd;
      dg += gnd * sc1 + gn * tsc;
      db += g1 * tsc;
    }
    if (a.d_scale) stf<T>(static_cast<T *>(a.d_scale) + i, d_scale);
  }
  // d_gamma / d_beta are zeroed by the caller (they share the zero-filled buffer of the column sums)
  atomicAdd(a.d_gamma + c, dg);
  if (a.d_beta) atomicAdd(a.d_beta + c, db);
}

// ---- gated residual on a (primal, tangent) pair in one pass each way.
//   forward   z = x + m g y,   tz = tx + m (g ty + tg y)                      (tx, ty, tg may be absent)
//   backward  from cotangents gz on z and gtz on tz (either may be absent; the skip gradients are gz and gtz themselves):
//             d_y = m (g gz + tg gtz),  d_ty = m g gtz,  d_g[b] += sum_s m (y gz + ty gtz),  d_tg[b] += sum_s m y gtz
struct GateDualArgs {
  const void *x, *tx, *y, *ty, *gate, *tgate, *mask;
  int64_t gate_stride, tgate_stride;
  void *z, *tz;
  const void *gz, *gtz;
  void *d_y, *d_ty;
  float *sums;  // [2, B, C]: gate, tgate
  int B, S, C;
  DropArgs drop;
};

template <typename T>
__global__ void __launch_bounds__(256) gated_dual_fwd_kernel(GateDualArgs a) {
  const int64_t total = (int64_t)a.B * a.S * a.C / 8;
  for (int64_t i8 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i8 < total; i8 += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = i8 * 8;
    const int c0 = (int)(e % a.C);
    const int b = (int)(e / ((int64_t)a.S * a.C));
    float xv[8], txv[8], yv[8], tyv[8], gv[8], tgv[8], mv[8], o[8], to[8];
    load8<T>(static_cast<const T *>(a.x) + e, xv);
    load8<T>(static_cast<const T *>(a.y) + e, yv);
    load8<T>(static_cast<const T *>(a.gate) + (int64_t)b * a.gate_stride + c0, gv);
    if (a.tx) load8<T>(static_cast<const T *>(a.tx) + e, txv);
    if (a.ty) load8<T>(static_cast<const T *>(a.ty) + e, tyv);
    if (a.tgate) load8<T>(static_cast<const T *>(a.tgate) + (int64_t)b * a.tgate_stride + c0, tgv);
    if (a.mask) load8<T>(static_cast<const T *>(a.mask) + e, mv);
    else if (a.drop.seed) dropout8(a.drop, i8, mv);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float m = (a.mask || a.drop.seed) ? mv[i] : 1.f;
      o[i] = xv[i] + m * gv[i] * yv[i];
      float br = 0.f;
      if (a.ty) br += gv[i] * tyv[i];
      if (a.tgate) br += tgv[i] * yv[i];
      to[i] = (a.tx ? txv[i] : 0.f) + m * br;
    }
    store8<T>(static_cast<T *>(a.z) + e, o);
    store8<T>(static_cast<T *>(a.tz) + e, to);
  }
}

// One thread owns 8 adjacent channels of `rows_per_cta` rows of one sample: the column sums stay in registers and leave
// with one atomic per channel and CTA; adjacent threads read adjacent 16-byte pieces of a row.
template <typename T>
__global__ void __launch_bounds__(128) gated_dual_bwd_kernel(GateDualArgs a, int rows_per_cta) {
  const int c0 = threadIdx.x * 8;
  if (c0 >= a.C) return;
  const int ctas_per_sample = (a.S + rows_per_cta - 1) / rows_per_cta;
  const int b = blockIdx.x / ctas_per_sample;
  const int s0 = (blockIdx.x % ctas_per_sample) * rows_per_cta;
  float gt[8], tgt[8], sg[8] = {}, stg[8] = {};
  load8<T>(static_cast<const T *>(a.gate) + (int64_t)b * a.gate_stride + c0, gt);
  if (a.tgate) load8<T>(static_cast<const T *>(a.tgate) + (int64_t)b * a.tgate_stride + c0, tgt);
  const int s1 = min(a.S, s0 + rows_per_cta);
#pragma unroll 2
  for (int s = s0; s < s1; ++s) {
    const int64_t e = ((int64_t)b * a.S + s) * a.C + c0;
    float yv[8], tyv[8], mv[8], g1[8], g2[8], o1[8], o2[8];
    load8<T>(static_cast<const T *>(a.y) + e, yv);
    if (a.gz) load8<T>(static_cast<const T *>(a.gz) + e, g1);
    if (a.gtz) load8<T>(static_cast<const T *>(a.gtz) + e, g2);
    if (a.ty && a.gtz) load8<T>(static_cast<const T *>(a.ty) + e, tyv);
    if (a.mask) load8<T>(static_cast<const T *>(a.mask) + e, mv);
    else if (a.drop.seed) dropout8(a.drop, e / 8, mv);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float m = (a.mask || a.drop.seed) ? mv[i] : 1.f;
      const float mg1 = a.gz ? m * g1[i] : 0.f, mg2 = a.gtz ? m * g2[i] : 0.f;
      o1[i] = gt[i] * mg1 + (a.tgate ? tgt[i] * mg2 : 0.f);
      o2[i] = gt[i] * mg2;
      sg[i] += yv[i] * mg1 + (a.ty && a.gtz ? tyv[i] * mg2 : 0.f);
      stg[i] += yv[i] * mg2;
    }
    store8<T>(static_cast<T *>(a.d_y) + e, o1);
    if (a.d_ty) store8<T>(static_cast<T *>(a.d_ty) + e, o2);
  }
  float *dg = a.sums + (int64_t)b * a.C + c0, *dtg = a.sums + ((int64_t)a.B + b) * a.C + c0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    atomicAdd(dg + i, sg[i]);
    if (a.gtz) atomicAdd(dtg + i, stg[i]);
  }
}

// ------------------------------------------------------------------------------------------------ GELU (tanh form)
// g(h) = h/2 (1 + tanh u), u = k (h + a h^3).  The MLP of the block (duo.py:118-123) applies it to a (primal, tangent)
// pair; with T = tanh u, u' = k (1 + 3 a h^2), u'' = 6 a k h:
//   g'  = (1 + T) / 2 + h/2 (1 - T^2) u'
//   g'' = (1 - T^2) (u' + h/2 (u'' - 2 T u'^2))
// mode 0: y = g(h);  mode 1: out = g'(h) * v (the tangent, and the VJP of either output with respect to its own input);
// mode 2: out = g'(h) * v and out2 = g''(h) * w * v (the VJP of the tangent output: with respect to the tangent and to h);
// mode 3: out = g(h) and out2 = g'(h) * v (primal and tangent in one pass);
// mode 4: out = g'(h) * v + g''(h) * w * u and out2 = g'(h) * u (both cotangents in one pass: v on y, u on ty, w = tangent
//         of h; out = gradient of h, out2 = gradient of the tangent).
struct GeluTerms {
  float g, d1, d2;
};
__device__ __forceinline__ GeluTerms gelu_terms(float h) {
  constexpr float k = 0.7978845608028654f, a = 0.044715f;
  const float h2 = h * h, T = tanhf(k * (h + a * h2 * h));
  const float up = k * (1.f + 3.f * a * h2), upp = 6.f * a * k * h, sech2 = 1.f - T * T;
  GeluTerms r;
  r.g = 0.5f * h * (1.f + T);
  r.d1 = 0.5f * (1.f + T) + 0.5f * h * sech2 * up;
  r.d2 = sech2 * (up + 0.5f * h * (upp - 2.f * T * up * up));
  return r;
}

template <typename T, int kMode>
__global__ void __launch_bounds__(256) gelu_dual_kernel(const T *h, const T *v, const T *w, const T *u, T *out, T *out2,
                                                        int64_t n8) {
  // two chunks per iteration: all loads of both are issued before the arithmetic, so every thread keeps two 16-byte
  // loads per operand in flight (one was not enough to cover the memory latency at full occupancy)
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i0 = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i0 < n8; i0 += 2 * stride) {
    const int64_t idx[2] = {i0, i0 + stride};
    float hv[2][8], vv[2][8], wv[2][8], uv[2][8];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      if (idx[c] >= n8) continue;
      load8<T>(h + idx[c] * 8, hv[c]);
      if (kMode >= 1) load8<T>(v + idx[c] * 8, vv[c]);
      if (kMode == 2 || kMode == 4) load8<T>(w + idx[c] * 8, wv[c]);
      if (kMode == 4) load8<T>(u + idx[c] * 8, uv[c]);
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      if (idx[c] >= n8) continue;
      float o[8], o2[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const GeluTerms t = gelu_terms(hv[c][j]);
        if (kMode == 0) o[j] = t.g;
        if (kMode == 1) o[j] = t.d1 * vv[c][j];
        if (kMode == 2) o[j] = t.d1 * vv[c][j], o2[j] = t.d2 * wv[c][j] * vv[c][j];
        if (kMode == 3) o[j] = t.g, o2[j] = t.d1 * vv[c][j];
        if (kMode == 4) o[j] = t.d1 * vv[c][j] + t.d2 * wv[c][j] * uv[c][j], o2[j] = t.d1 * uv[c][j];
      }
      store8<T>(out + idx[c] * 8, o);
      if (kMode >= 2) store8<T>(out2 + idx[c] * 8, o2);
    }
  }
}

// Calls f(T{}, integral_constant<NV>) for the element type (dtype code 0 = bf16, 2 = fp32) and C / 256 in 1..4.
template <typename F>
cudaError_t dispatch(int dtype, int C, F &&f) {
  auto with_nv = [&](auto t) -> cudaError_t {
    switch (C / 256) {
      case 1: return f(t, std::integral_constant<int, 1>{});
      case 2: return f(t, std::integral_constant<int, 2>{});
      case 3: return f(t, std::integral_constant<int, 3>{});
      case 4: return f(t, std::integral_constant<int, 4>{});
      default: return cudaErrorInvalidValue;
    }
  };
  if (dtype == JVPATTN_BF16) return with_nv(__nv_bfloat16{});
  if (dtype == JVPATTN_FP32) return with_nv(float{});
  return cudaErrorInvalidValue;
}

}  // namespace

bool dual_shape_ok(int B, int S, int C) { return B >= 0 && S >= 1 && C >= 256 && C <= 1024 && C % 256 == 0; }

cudaError_t ln_modulate(int which, const void *x, const void *tx, const float *gamma, const float *beta, const void *shift,
                        const void *scale, const void *tshift, const void *tscale, int64_t mod_stride, int64_t tmod_stride,
                        float *mean, float *rstd, void *out, const void *g, void *dx, void *dtx, float *sums, int B, int S, int C,
                        float eps, int exact, int dtype, cudaStream_t stream) {
  LnArgs a{x, tx, gamma, beta, shift, scale, tshift, tscale, mod_stride, tmod_stride, mean, rstd, out, g, dx, dtx, sums, B, S, C, eps, exact};
  const int64_t rows = (int64_t)B * S;
  if (rows == 0) return cudaSuccess;
  LaunchScope scope(kIdDual, stream);
  return dispatch(dtype, C, [&](auto t, auto nv) -> cudaError_t {
    using T = decltype(t);
    constexpr int NV = decltype(nv)::value;
    if (which == 0 || which == 1) {
      const unsigned grid = (unsigned)((rows + kWarpsPerCta - 1) / kWarpsPerCta);
      if (which == 0) ln_modulate_fwd_kernel<T, NV, false><<<grid, kWarpsPerCta * 32, 0, stream>>>(a);
      else ln_modulate_fwd_kernel<T, NV, true><<<grid, kWarpsPerCta * 32, 0, stream>>>(a);
    } else {
      const int rows_cta = rows_per_cta(B, S, 16);
      const unsigned grid = (unsigned)(B * ((S + rows_cta - 1) / rows_cta));
      if (which == 2) {
        ln_modulate_bwd_kernel<T, NV><<<grid, kWarpsPerCta * 32, kWarpsPerCta * 2 * NV * 256 * 4, stream>>>(a, rows_cta);
      } else {
        auto k = ln_modulate_bwd_tangent_kernel<T, NV>;
        constexpr int smem = kWarpsPerCta * 3 * NV * 256 * 4;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        k<<<grid, kWarpsPerCta * 32, smem, stream>>>(a, rows_cta);
      }
    }
    return cudaGetLastError();
  });
}

cudaError_t gated_residual(const void *x, const void *y, const void *gate, const void *mask, int64_t gate_stride, void *z, int B,
                           int S, int C, int dtype, const unsigned long long *drop_seed, unsigned drop_call, float drop_p,
                           cudaStream_t stream) {
  const int64_t total = (int64_t)B * S * C / 8;
  if (total == 0) return cudaSuccess;
  if (C % 8) return cudaErrorInvalidValue;
  GateArgs a{x, y, gate, mask, gate_stride, z, B, S, C, {drop_seed, drop_call, drop_p}};
  LaunchScope scope(kIdDual, stream);
  const unsigned grid = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 8);
  if (dtype == JVPATTN_BF16) gated_residual_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(a);
  else if (dtype == JVPATTN_FP32) gated_residual_fwd_kernel<float><<<grid, 256, 0, stream>>>(a);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t ln_finalize(const float *p, const float *t, const float *gamma, const float *beta, const void *scale,
                        const void *tscale, int64_t mod_stride, int64_t tmod_stride, void *d_shift, void *d_scale, void *d_tshift,
                        void *d_tscale, float *d_gamma, float *d_beta, int B, int C, int dtype, cudaStream_t stream) {
  if (C == 0) return cudaSuccess;
  LnFinalArgs a{p, t, gamma, beta, scale, tscale, mod_stride, tmod_stride, d_shift, d_scale, d_tshift, d_tscale, d_gamma, d_beta, B, C};
  LaunchScope scope(kIdDual, stream);
  if (B == 0) return cudaSuccess;
  const dim3 grid((unsigned)((C + 127) / 128), (unsigned)((B + kFinalSamples - 1) / kFinalSamples));
  if (dtype == JVPATTN_BF16) ln_finalize_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(a);
  else if (dtype == JVPATTN_FP32) ln_finalize_kernel<float><<<grid, 128, 0, stream>>>(a);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t gated_residual_dual(int which, const void *x, const void *tx, const void *y, const void *ty, const void *gate,
                                const void *tgate, const void *mask, int64_t gate_stride, int64_t tgate_stride, void *z, void *tz,
                                const void *gz, const void *gtz, void *d_y, void *d_ty, float *sums, int B, int S, int C, int dtype,
                                const unsigned long long *drop_seed, unsigned drop_call, float drop_p, cudaStream_t stream) {
  if ((int64_t)B * S * C == 0) return cudaSuccess;
  if (C % 8 || C > 1024) return cudaErrorInvalidValue;
  GateDualArgs a{x, tx, y, ty, gate, tgate, mask, gate_stride, tgate_stride, z, tz, gz, gtz, d_y, d_ty, sums, B, S, C,
                 {drop_seed, drop_call, drop_p}};
  LaunchScope scope(kIdDual, stream);
  auto launch = [&](auto tag) -> cudaError_t {
    using T = decltype(tag);
    if (which == 0) {
      const int64_t n8 = (int64_t)B * S * C / 8;
      gated_dual_fwd_kernel<T><<<(unsigned)std::min<int64_t>((n8 + 255) / 256, 148 * 16), 256, 0, stream>>>(a);
    } else {
      const int rows_cta = rows_per_cta(B, S, 8);
      gated_dual_bwd_kernel<T><<<(unsigned)(B * ((S + rows_cta - 1) / rows_cta)), 128, 0, stream>>>(a, rows_cta);
    }
    return cudaGetLastError();
  };
  if (dtype == JVPATTN_BF16) return launch(__nv_bfloat16{});
  if (dtype == JVPATTN_FP32) return launch(float{});
  return cudaErrorInvalidValue;
}

cudaError_t gelu_dual(int mode, const void *h, const void *v, const void *w, const void *u, void *out, void *out2, int64_t n,
                      int dtype, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  if (n % 8) return cudaErrorInvalidValue;
  const int64_t n8 = n / 8;
  const unsigned grid = (unsigned)std::min<int64_t>((n8 + 511) / 512, 148 * 8);
  LaunchScope scope(kIdDual, stream);
  auto launch = [&](auto tag) -> cudaError_t {
    using T = decltype(tag);
    auto H = static_cast<const T *>(h), V = static_cast<const T *>(v), W = static_cast<const T *>(w), U = static_cast<const T *>(u);
    auto O = static_cast<T *>(out), O2 = static_cast<T *>(out2);
    switch (mode) {
      case 0: gelu_dual_kernel<T, 0><<<grid, 256, 0, stream>>>(H, V, W, U, O, O2, n8); break;
      case 1: gelu_dual_kernel<T, 1><<<grid, 256, 0, stream>>>(H, V, W, U, O, O2, n8); break;
      case 2: gelu_dual_kernel<T, 2><<<grid, 256, 0, stream>>>(H, V, W, U, O, O2, n8); break;
      case 3: gelu_dual_kernel<T, 3><<<grid, 256, 0, stream>>>(H, V, W, U, O, O2, n8); break;
      case 4: gelu_dual_kernel<T, 4><<<grid, 256, 0, stream>>>(H, V, W, U, O, O2, n8); break;
      default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
  };
  if (dtype == JVPATTN_BF16) return launch(__nv_bfloat16{});
  if (dtype == JVPATTN_FP32) return launch(float{});
  return cudaErrorInvalidValue;
}

}  // namespace jvpattn
