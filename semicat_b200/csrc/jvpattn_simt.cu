// Portable SIMT kernels for the attention JVP forward and backward.
//
// These cover every shape the interface accepts (any len_q / len_k, head_dim 16..128, bf16 or fp16,
// arbitrary batch/head/row strides) with plain fp32 FMA arithmetic.  They are the kernels AUTO
// falls back to for shapes the tcgen05 kernels do not take, and the on-device cross-check for them.
// One warp owns one output row; key/value (forward, dq) or query (dk, dv) tiles of 32 rows are
// staged in shared memory and shared by the 8 warps of a block.
//
// Algorithm: online-softmax form of semicat/jvp_utils/ryu_triton.py:198-291 (forward) and the
// closed form of the six VJPs that semicat/jvp_utils/flash_jvp_backward.py and
// semicat/jvp_utils/flash_attn_triton.py:406-685 compute (backward).
#include "jvpattn_common.cuh"

namespace jvpattn {
namespace {

constexpr int kTile = 32;   // rows of the shared tile (one per lane)
constexpr int kWarps = 8;
constexpr int kRowsPerWarp = 2;
constexpr int kRows = kWarps * kRowsPerWarp;
constexpr int kMaxReg = 4;  // head_dim <= 128 -> at most 4 channels per lane

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}

// Cooperative load of `kTile` rows [row0, row0+kTile) of a view into a padded shared tile; rows beyond
// `len` are zero.
template <typename T>
__device__ __forceinline__ void load_tile(T *dst, const View &v, int b, int h, int row0, int len, int D, int DP) {
  const T *base = static_cast<const T *>(v.ptr);
  for (int idx = threadIdx.x; idx < kTile * D; idx += blockDim.x) {
    int j = idx / D, dd = idx - j * D;
    int row = row0 + j;
    dst[j * DP + dd] = row < len ? base[v.offset(b, h, row) + dd] : Elem<T>::from_f(0.f);
  }
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32) simt_fwd_kernel(FwdArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = a.D, DP = D + 2;
  T *Ks = reinterpret_cast<T *>(smem_raw);
  T *Kd = Ks + kTile * DP;
  T *Vs = Kd + kTile * DP;
  T *Vd = Vs + kTile * DP;
  float *rows = reinterpret_cast<float *>(Vd + kTile * DP);  // [warp][r][2][D]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int row0 = blockIdx.x * kRows + warp * kRowsPerWarp;
  float *myrows = rows + (size_t)warp * kRowsPerWarp * 2 * D;

  const T *qp = static_cast<const T *>(a.q.ptr);
  const T *tqp = static_cast<const T *>(a.tq.ptr);
  for (int r = 0; r < kRowsPerWarp; ++r) {
    int row = row0 + r;
    for (int dd = lane; dd < D; dd += 32) {
      bool ok = row < a.Lq;
      myrows[(r * 2 + 0) * D + dd] = ok ? Elem<T>::to_f(qp[a.q.offset(b, h, row) + dd]) : 0.f;
      myrows[(r * 2 + 1) * D + dd] = ok ? Elem<T>::to_f(tqp[a.tq.offset(b, h, row) + dd]) : 0.f;
    }
  }

  float m[kRowsPerWarp], l[kRowsPerWarp], mu[kRowsPerWarp];
  float acc[kRowsPerWarp][kMaxReg], gacc[kRowsPerWarp][kMaxReg];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    m[r] = -INFINITY; l[r] = 0.f; mu[r] = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxReg; ++i) { acc[r][i] = 0.f; gacc[r][i] = 0.f; }
  }

  for (int kv0 = 0; kv0 < a.Lk; kv0 += kTile) {
    __syncthreads();
    load_tile<T>(Ks, a.k, b, h, kv0, a.Lk, D, DP);
    load_tile<T>(Kd, a.tk, b, h, kv0, a.Lk, D, DP);
    load_tile<T>(Vs, a.v, b, h, kv0, a.Lk, D, DP);
    load_tile<T>(Vd, a.tv, b, h, kv0, a.Lk, D, DP);
    __syncthreads();
    const bool valid = kv0 + lane < a.Lk;
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      const float *qr = myrows + (r * 2 + 0) * D;
      const float *tqr = myrows + (r * 2 + 1) * D;
      float s = 0.f, sd = 0.f;
      for (int dd = 0; dd < D; ++dd) {
        float kk = Elem<T>::to_f(Ks[lane * DP + dd]);
        float kd = Elem<T>::to_f(Kd[lane * DP + dd]);
        s = fmaf(qr[dd], kk, s);
        sd = fmaf(tqr[dd], kk, fmaf(qr[dd], kd, sd));
      }
      s = valid ? s * a.scale : -INFINITY;
      sd *= a.scale;
      float m_new = fmaxf(m[r], warp_max(s));
      float alpha = __expf(m[r] - m_new);  // exp(-inf) = 0 on the first tile
      float p = valid ? __expf(s - m_new) : 0.f;
      float u = p * sd;
      l[r] = l[r] * alpha + warp_sum(p);
      mu[r] = mu[r] * alpha + warp_sum(u);
      m[r] = m_new;
#pragma unroll
      for (int i = 0; i < kMaxReg; ++i) { acc[r][i] *= alpha; gacc[r][i] *= alpha; }
      for (int j = 0; j < kTile; ++j) {
        float pj = __shfl_sync(0xffffffffu, p, j);
        float uj = __shfl_sync(0xffffffffu, u, j);
#pragma unroll
        for (int i = 0; i < kMaxReg; ++i) {
          int dd = lane + 32 * i;
          if (dd < D) {
            float vv = Elem<T>::to_f(Vs[j * DP + dd]);
            float vd = Elem<T>::to_f(Vd[j * DP + dd]);
            acc[r][i] = fmaf(pj, vv, acc[r][i]);
            gacc[r][i] = fmaf(uj, vv, fmaf(pj, vd, gacc[r][i]));
          }
        }
      }
    }
  }

  T *op = static_cast<T *>(a.o.ptr);
  T *top = static_cast<T *>(a.to.ptr);
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    int row = row0 + r;
    if (row >= a.Lq) continue;
    float inv = 1.f / l[r];
    float mun = mu[r] * inv;
#pragma unroll
    for (int i = 0; i < kMaxReg; ++i) {
      int dd = lane + 32 * i;
      if (dd < D) {
        float o = acc[r][i] * inv;
        op[a.o.offset(b, h, row) + dd] = Elem<T>::from_f(o);
        if (top) top[a.to.offset(b, h, row) + dd] = Elem<T>::from_f(gacc[r][i] * inv - mun * o);  // null: primal only
      }
    }
    if (lane == 0) {
      size_t si = ((size_t)b * a.H + h) * a.stat_len + row;
      a.lse[si] = m[r] + __logf(l[r]);
      if (a.mu) a.mu[si] = mun;
      if (a.li) a.li[si] = l[r];
    }
  }
}

// dq and dtq: one warp per query row, loops over key/value tiles.
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) simt_bwd_q_kernel(BwdArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = a.D, DP = D + 2;
  T *Ks = reinterpret_cast<T *>(smem_raw);
  T *Kd = Ks + kTile * DP;
  T *Vs = Kd + kTile * DP;
  T *Vd = Vs + kTile * DP;
  float *rows = reinterpret_cast<float *>(Vd + kTile * DP);  // [warp][r][4][D]: q, tq, G, gO

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int row0 = blockIdx.x * kRows + warp * kRowsPerWarp;
  float *myrows = rows + (size_t)warp * kRowsPerWarp * 4 * D;
  const bool has_t = a.g_to.ptr != nullptr, has_o = a.g_o.ptr != nullptr;

  float lse[kRowsPerWarp], mu[kRowsPerWarp], delta[kRowsPerWarp], deltad[kRowsPerWarp], delta0[kRowsPerWarp];
  for (int r = 0; r < kRowsPerWarp; ++r) {
    int row = row0 + r;
    bool ok = row < a.Lq;
    float d1 = 0.f, d2 = 0.f, d3 = 0.f;
    for (int dd = lane; dd < D; dd += 32) {
      float q = 0.f, tq = 0.f, g = 0.f, go = 0.f, o = 0.f, to = 0.f;
      if (ok) {
        q = Elem<T>::to_f(static_cast<const T *>(a.q.ptr)[a.q.offset(b, h, row) + dd]);
        tq = Elem<T>::to_f(static_cast<const T *>(a.tq.ptr)[a.tq.offset(b, h, row) + dd]);
        o = Elem<T>::to_f(static_cast<const T *>(a.o.ptr)[a.o.offset(b, h, row) + dd]);
        to = Elem<T>::to_f(static_cast<const T *>(a.to.ptr)[a.to.offset(b, h, row) + dd]);
        if (has_t) g = Elem<T>::to_f(static_cast<const T *>(a.g_to.ptr)[a.g_to.offset(b, h, row) + dd]);
        if (has_o) go = Elem<T>::to_f(static_cast<const T *>(a.g_o.ptr)[a.g_o.offset(b, h, row) + dd]);
      }
      myrows[(r * 4 + 0) * D + dd] = q;
      myrows[(r * 4 + 1) * D + dd] = tq;
      myrows[(r * 4 + 2) * D + dd] = g;
      myrows[(r * 4 + 3) * D + dd] = go;
      d1 = fmaf(g, o, d1);
      d2 = fmaf(g, to, d2);
      d3 = fmaf(go, o, d3);
    }
    delta[r] = warp_sum(d1);
    deltad[r] = warp_sum(d2);
    delta0[r] = warp_sum(d3);
    size_t si = ((size_t)b * a.H + h) * a.stat_len + (ok ? row : 0);
    lse[r] = a.lse[si];
    mu[r] = a.mu[si];
  }

  float dq[kRowsPerWarp][kMaxReg], dtq[kRowsPerWarp][kMaxReg];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
    for (int i = 0; i < kMaxReg; ++i) { dq[r][i] = 0.f; dtq[r][i] = 0.f; }

  for (int kv0 = 0; kv0 < a.Lk; kv0 += kTile) {
    __syncthreads();
    load_tile<T>(Ks, a.k, b, h, kv0, a.Lk, D, DP);
    load_tile<T>(Kd, a.tk, b, h, kv0, a.Lk, D, DP);
    load_tile<T>(Vs, a.v, b, h, kv0, a.Lk, D, DP);
    load_tile<T>(Vd, a.tv, b, h, kv0, a.Lk, D, DP);
    __syncthreads();
    const bool valid = kv0 + lane < a.Lk;
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      const float *qr = myrows + (r * 4 + 0) * D, *tqr = myrows + (r * 4 + 1) * D;
      const float *gr = myrows + (r * 4 + 2) * D, *gor = myrows + (r * 4 + 3) * D;
      float s = 0.f, sd = 0.f, aa = 0.f, bm = 0.f, a0 = 0.f;
      for (int dd = 0; dd < D; ++dd) {
        float kk = Elem<T>::to_f(Ks[lane * DP + dd]), kd = Elem<T>::to_f(Kd[lane * DP + dd]);
        float vv = Elem<T>::to_f(Vs[lane * DP + dd]), vd = Elem<T>::to_f(Vd[lane * DP + dd]);
        s = fmaf(qr[dd], kk, s);
        sd = fmaf(tqr[dd], kk, fmaf(qr[dd], kd, sd));
        aa = fmaf(gr[dd], vv, aa);
        bm = fmaf(gr[dd], vd, bm);
        a0 = fmaf(gor[dd], vv, a0);
      }
      float p = valid ? __expf(s * a.scale - lse[r]) : 0.f;
      float n = sd * a.scale - mu[r];
      float w1 = a.scale * p * (aa - delta[r]);
      float w2 = a.scale * p * ((aa - delta[r]) * n + bm - deltad[r] + a0 - delta0[r]);
      for (int j = 0; j < kTile; ++j) {
        float w1j = __shfl_sync(0xffffffffu, w1, j);
        float w2j = __shfl_sync(0xffffffffu, w2, j);
#pragma unroll
        for (int i = 0; i < kMaxReg; ++i) {
          int dd = lane + 32 * i;
          if (dd < D) {
            float kk = Elem<T>::to_f(Ks[j * DP + dd]), kd = Elem<T>::to_f(Kd[j * DP + dd]);
            dtq[r][i] = fmaf(w1j, kk, dtq[r][i]);
            dq[r][i] = fmaf(w1j, kd, fmaf(w2j, kk, dq[r][i]));
          }
        }
      }
    }
  }

#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    int row = row0 + r;
    if (row >= a.Lq) continue;
#pragma unroll
    for (int i = 0; i < kMaxReg; ++i) {
      int dd = lane + 32 * i;
      if (dd < D) {
        static_cast<T *>(a.dq.ptr)[a.dq.offset(b, h, row) + dd] = Elem<T>::from_f(dq[r][i]);
        if (has_t) static_cast<T *>(a.dtq.ptr)[a.dtq.offset(b, h, row) + dd] = Elem<T>::from_f(dtq[r][i]);
      }
    }
  }
}

// dk, dv, dtk, dtv: one warp per key row, loops over query tiles.
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) simt_bwd_kv_kernel(BwdArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = a.D, DP = D + 2;
  T *Qs = reinterpret_cast<T *>(smem_raw);
  T *Qd = Qs + kTile * DP;
  T *Gs = Qd + kTile * DP;
  T *Go = Gs + kTile * DP;
  float *stats = reinterpret_cast<float *>(Go + kTile * DP);  // [5][kTile]: lse, mu, delta, deltad, delta0
  float *rows = stats + 5 * kTile;                            // [warp][r][4][D]: k, tk, v, tv

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int row0 = blockIdx.x * kRows + warp * kRowsPerWarp;
  float *myrows = rows + (size_t)warp * kRowsPerWarp * 4 * D;
  const bool has_t = a.g_to.ptr != nullptr, has_o = a.g_o.ptr != nullptr;

  for (int r = 0; r < kRowsPerWarp; ++r) {
    int row = row0 + r;
    bool ok = row < a.Lk;
    for (int dd = lane; dd < D; dd += 32) {
      myrows[(r * 4 + 0) * D + dd] = ok ? Elem<T>::to_f(static_cast<const T *>(a.k.ptr)[a.k.offset(b, h, row) + dd]) : 0.f;
      myrows[(r * 4 + 1) * D + dd] = ok ? Elem<T>::to_f(static_cast<const T *>(a.tk.ptr)[a.tk.offset(b, h, row) + dd]) : 0.f;
      myrows[(r * 4 + 2) * D + dd] = ok ? Elem<T>::to_f(static_cast<const T *>(a.v.ptr)[a.v.offset(b, h, row) + dd]) : 0.f;
      myrows[(r * 4 + 3) * D + dd] = ok ? Elem<T>::to_f(static_cast<const T *>(a.tv.ptr)[a.tv.offset(b, h, row) + dd]) : 0.f;
    }
  }

  float dk[kRowsPerWarp][kMaxReg], dtk[kRowsPerWarp][kMaxReg], dv[kRowsPerWarp][kMaxReg], dtv[kRowsPerWarp][kMaxReg];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
    for (int i = 0; i < kMaxReg; ++i) { dk[r][i] = 0.f; dtk[r][i] = 0.f; dv[r][i] = 0.f; dtv[r][i] = 0.f; }

  for (int q0 = 0; q0 < a.Lq; q0 += kTile) {
    __syncthreads();
    load_tile<T>(Qs, a.q, b, h, q0, a.Lq, D, DP);
    load_tile<T>(Qd, a.tq, b, h, q0, a.Lq, D, DP);
    if (has_t) load_tile<T>(Gs, a.g_to, b, h, q0, a.Lq, D, DP);
    if (has_o) load_tile<T>(Go, a.g_o, b, h, q0, a.Lq, D, DP);
    // row statistics of this query tile: each warp takes rows warp, warp+8, ...
    for (int j = warp; j < kTile; j += kWarps) {
      int row = q0 + j;
      bool ok = row < a.Lq;
      float d1 = 0.f, d2 = 0.f, d3 = 0.f;
      if (ok) {
        for (int dd = lane; dd < D; dd += 32) {
          float o = Elem<T>::to_f(static_cast<const T *>(a.o.ptr)[a.o.offset(b, h, row) + dd]);
          float to = Elem<T>::to_f(static_cast<const T *>(a.to.ptr)[a.to.offset(b, h, row) + dd]);
          float g = has_t ? Elem<T>::to_f(static_cast<const T *>(a.g_to.ptr)[a.g_to.offset(b, h, row) + dd]) : 0.f;
          float go = has_o ? Elem<T>::to_f(static_cast<const T *>(a.g_o.ptr)[a.g_o.offset(b, h, row) + dd]) : 0.f;
          d1 = fmaf(g, o, d1);
          d2 = fmaf(g, to, d2);
          d3 = fmaf(go, o, d3);
        }
      }
      d1 = warp_sum(d1); d2 = warp_sum(d2); d3 = warp_sum(d3);
      if (lane == 0) {
        size_t si = ((size_t)b * a.H + h) * a.stat_len + (ok ? row : 0);
        stats[0 * kTile + j] = ok ? a.lse[si] : INFINITY;  // exp(s - inf) = 0 for padded rows
        stats[1 * kTile + j] = ok ? a.mu[si] : 0.f;
        stats[2 * kTile + j] = d1;
        stats[3 * kTile + j] = d2;
        stats[4 * kTile + j] = d3;
      }
    }
    __syncthreads();
    const bool valid = q0 + lane < a.Lq;
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      const float *kr = myrows + (r * 4 + 0) * D, *tkr = myrows + (r * 4 + 1) * D;
      const float *vr = myrows + (r * 4 + 2) * D, *tvr = myrows + (r * 4 + 3) * D;
      float s = 0.f, sd = 0.f, aa = 0.f, bm = 0.f, a0 = 0.f;
      for (int dd = 0; dd < D; ++dd) {
        float qq = Elem<T>::to_f(Qs[lane * DP + dd]), qd = Elem<T>::to_f(Qd[lane * DP + dd]);
        s = fmaf(qq, kr[dd], s);
        sd = fmaf(qd, kr[dd], fmaf(qq, tkr[dd], sd));
        if (has_t) {
          float g = Elem<T>::to_f(Gs[lane * DP + dd]);
          aa = fmaf(g, vr[dd], aa);
          bm = fmaf(g, tvr[dd], bm);
        }
        if (has_o) a0 = fmaf(Elem<T>::to_f(Go[lane * DP + dd]), vr[dd], a0);
      }
      float p = valid ? __expf(s * a.scale - stats[lane]) : 0.f;
      float n = sd * a.scale - stats[kTile + lane];
      float da = aa - stats[2 * kTile + lane];
      float w1 = a.scale * p * da;
      float w2 = a.scale * p * (da * n + bm - stats[3 * kTile + lane] + a0 - stats[4 * kTile + lane]);
      float pd = p * n;
      for (int j = 0; j < kTile; ++j) {
        float w1j = __shfl_sync(0xffffffffu, w1, j);
        float w2j = __shfl_sync(0xffffffffu, w2, j);
        float pj = __shfl_sync(0xffffffffu, p, j);
        float pdj = __shfl_sync(0xffffffffu, pd, j);
#pragma unroll
        for (int i = 0; i < kMaxReg; ++i) {
          int dd = lane + 32 * i;
          if (dd < D) {
            float qq = Elem<T>::to_f(Qs[j * DP + dd]), qd = Elem<T>::to_f(Qd[j * DP + dd]);
            float g = has_t ? Elem<T>::to_f(Gs[j * DP + dd]) : 0.f;
            float go = has_o ? Elem<T>::to_f(Go[j * DP + dd]) : 0.f;
            dtk[r][i] = fmaf(w1j, qq, dtk[r][i]);
            dk[r][i] = fmaf(w1j, qd, fmaf(w2j, qq, dk[r][i]));
            dtv[r][i] = fmaf(pj, g, dtv[r][i]);
            dv[r][i] = fmaf(pdj, g, fmaf(pj, go, dv[r][i]));
          }
        }
      }
    }
  }

#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    int row = row0 + r;
    if (row >= a.Lk) continue;
#pragma unroll
    for (int i = 0; i < kMaxReg; ++i) {
      int dd = lane + 32 * i;
      if (dd < D) {
        static_cast<T *>(a.dk.ptr)[a.dk.offset(b, h, row) + dd] = Elem<T>::from_f(dk[r][i]);
        static_cast<T *>(a.dv.ptr)[a.dv.offset(b, h, row) + dd] = Elem<T>::from_f(dv[r][i]);
        if (has_t) {
          static_cast<T *>(a.dtk.ptr)[a.dtk.offset(b, h, row) + dd] = Elem<T>::from_f(dtk[r][i]);
          static_cast<T *>(a.dtv.ptr)[a.dtv.offset(b, h, row) + dd] = Elem<T>::from_f(dtv[r][i]);
        }
      }
    }
  }
}

template <typename K, typename A>
cudaError_t launch(int id, K kernel, dim3 grid, size_t smem, const A &a, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  {
    LaunchScope scope(id, stream);
    kernel<<<grid, kWarps * 32, smem, stream>>>(a);
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t simt_fwd(const FwdArgs &a, cudaStream_t stream) {
  if (a.B == 0 || a.H == 0 || a.Lq == 0) return cudaSuccess;
  size_t esz = 2;
  size_t smem = 4 * kTile * (a.D + 2) * esz + (size_t)kWarps * kRowsPerWarp * 2 * a.D * sizeof(float);
  dim3 grid((a.Lq + kRows - 1) / kRows, a.H, a.B);
  return a.dtype == JVPATTN_BF16 ? launch(kIdFwdSimt, simt_fwd_kernel<__nv_bfloat16>, grid, smem, a, stream)
                                 : launch(kIdFwdSimt, simt_fwd_kernel<__half>, grid, smem, a, stream);
}

cudaError_t simt_bwd(const BwdArgs &a, cudaStream_t stream) {
  if (a.B == 0 || a.H == 0) return cudaSuccess;
  size_t esz = 2;
  size_t tile = 4 * kTile * (a.D + 2) * esz;
  size_t rows = (size_t)kWarps * kRowsPerWarp * 4 * a.D * sizeof(float);
  cudaError_t e = cudaSuccess;
  if (a.Lq > 0) {
    dim3 grid((a.Lq + kRows - 1) / kRows, a.H, a.B);
    e = a.dtype == JVPATTN_BF16 ? launch(kIdBwdQuerySimt, simt_bwd_q_kernel<__nv_bfloat16>, grid, tile + rows, a, stream)
                                : launch(kIdBwdQuerySimt, simt_bwd_q_kernel<__half>, grid, tile + rows, a, stream);
    if (e != cudaSuccess) return e;
  }
  if (a.Lk > 0) {
    dim3 grid((a.Lk + kRows - 1) / kRows, a.H, a.B);
    size_t smem = tile + 5 * kTile * sizeof(float) + rows;
    e = a.dtype == JVPATTN_BF16 ? launch(kIdBwdKeySimt, simt_bwd_kv_kernel<__nv_bfloat16>, grid, smem, a, stream)
                                : launch(kIdBwdKeySimt, simt_bwd_kv_kernel<__half>, grid, smem, a, stream);
  }
  return e;
}

}  // namespace jvpattn
