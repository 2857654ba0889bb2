// Fused attention-JVP forward for sm_100a: O = softmax(s) V and Od = (P o (sd - mu)) V + P Vd in one pass,
// tcgen05 MMAs accumulating in TMEM, TMA-staged operand tiles, online softmax.
//
// One CTA owns 128 query rows of one (batch, head) and walks the key axis in tiles of 64.
//   warp 0      TMA producer: Q, Qd once; K, Kd, V, Vd per key tile through a 2-stage ring
//   warp 1      MMA issuer (one elected thread): S = Q K^T, Sd = Qd K^T + Q Kd^T into TMEM, then
//               O += P V and Od' += U V + P Vd with P, U read back from TMEM as the A operand
//   warps 2..5  softmax: one thread per query row; reads S, Sd from TMEM, keeps the running max, sum and
//               mu, writes P = exp(s - m) and U = P o sd as 16-bit operands over the score columns
// Od' accumulates sum(P o sd) V + sum(P) Vd; the epilogue applies Od = Od'/l - (mu/l) O, the same
// algebra as the reference kernel (semicat/jvp_utils/ryu_triton.py:198-291).
//
// TMEM columns: [0,D) O, [D,2D) Od', [2D,2D+64) S / P, [2D+64,2D+128) Sd / U.  For D = 64 that is 256 columns
// and under 100 KB of shared memory, so two CTAs share an SM and one's MMAs overlap the other's softmax.
//
// kHasT = false is the primal-only instance (no tangents given): the same pipeline without Qd, Kd, Vd, Sd, U and Od,
// i.e. plain flash attention that writes O and lse.  It serves the callers' non-JVP attention (the reference uses
// F.scaled_dot_product_attention there, semicat/net/duo.py:143-152) so that one kernel family covers the whole step.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "jvpattn_common.cuh"
#include "sm100_attn.cuh"
#include "sm100_ptx.cuh"

namespace jvpattn {
namespace {

using namespace ptx;

constexpr int kBM = 128;     // query rows per CTA (= TMEM lanes)
constexpr int kBN = 64;      // keys per tile
constexpr int kStages = 2;
constexpr int kThreads = 192;
// Lazy rescale, in log2 units: the old reference maximum is kept while the new one is at most this far above it, so P
// stays below 2^threshold and O / Od' need no rescale.  bf16 has the exponent range for 2^8; fp16 operands do not
// (U = P o scale*sd would overflow for tangents 256 times smaller than with an exact maximum), so fp16 keeps the
// exact running maximum, as the reference kernel does (ryu_triton.py:229-231).
template <typename T> struct RescaleThreshold { static constexpr float value = 8.0f; };
template <> struct RescaleThreshold<__half> { static constexpr float value = 0.0f; };

template <int D>
struct FwdSmem {
  static constexpr int kBoxes = D / 64;
  alignas(1024) uint16_t q[kBoxes][kBM * 64];
  alignas(1024) uint16_t tq[kBoxes][kBM * 64];
  alignas(1024) uint16_t kv[kStages][4][kBoxes][kBN * 64];  // per stage: K, Kd, V, Vd (adjacent so pairs can be one operand)
  uint64_t q_full, kv_full[kStages], kv_empty[kStages], s_full, p_full, o_done;
  uint32_t tmem_base;
};

struct FwdMaps {
  CUtensorMap q, tq, k, tk, v, tv;
  CUtensorMap o, to;  // outputs as 128-row x 64-channel store boxes
};

template <int D, typename T, bool kHasT>
__global__ void __launch_bounds__(kThreads, D == 64 ? 2 : 1) sm100_fwd_kernel(const __grid_constant__ FwdMaps maps, FwdArgs a) {
  extern __shared__ unsigned char smem_raw[];
  using Smem = FwdSmem<D>;
  Smem &s = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kBoxes = D / 64;
  constexpr uint32_t kTmemCols = (2 * D + 128) <= 256 ? 256 : 512;
  constexpr uint32_t kColO = 0, kColOd = D, kColS = 2 * D, kColSd = 2 * D + 64;
  constexpr bool kBf16 = IsBf16<T>::value;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * kBM;
  const int ntiles = (a.Lk + kBN - 1) / kBN;

  if (threadIdx.x == 0) {
    mbar_init(&s.q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&s.kv_full[i], 1);
      mbar_init(&s.kv_empty[i], 1);
    }
    mbar_init(&s.s_full, 1);
    mbar_init(&s.p_full, 128);
    mbar_init(&s.o_done, 1);
    fence_barrier_init();
    // The barriers this thread just initialised are all the first requests need: the query rows and the first
    // key tiles are on their way while the other warps allocate tensor memory and meet at the barrier below.
    prefetch_tensormap(&maps.q);
    prefetch_tensormap(&maps.k);
    constexpr uint32_t kKvBytes = (kHasT ? 4 : 2) * kBN * D * 2;
    mbar_expect_tx(&s.q_full, (kHasT ? 2 : 1) * kBM * D * 2);
    for (int x = 0; x < kBoxes; ++x) {
      tma_load_4d(s.q[x], &maps.q, &s.q_full, 64 * x, q0, h, b);
      if (kHasT) tma_load_4d(s.tq[x], &maps.tq, &s.q_full, 64 * x, q0, h, b);
    }
    for (int j = 0; j < ntiles && j < kStages; ++j) {
      // (test hook: with `inject` the first tile's barrier expects 16 bytes that never arrive, so every role's wait
      //  on it, or on what follows from it, runs out and the CTA leaves through the normal teardown)
      mbar_expect_tx(&s.kv_full[j], kKvBytes + ((a.inject == 1 && j == 0) ? 16 : 0));
      for (int x = 0; x < kBoxes; ++x) {
        tma_load_4d(s.kv[j][0][x], &maps.k, &s.kv_full[j], 64 * x, j * kBN, h, b);
        if (kHasT) tma_load_4d(s.kv[j][1][x], &maps.tk, &s.kv_full[j], 64 * x, j * kBN, h, b);
        tma_load_4d(s.kv[j][2][x], &maps.v, &s.kv_full[j], 64 * x, j * kBN, h, b);
        if (kHasT) tma_load_4d(s.kv[j][3][x], &maps.tv, &s.kv_full[j], 64 * x, j * kBN, h, b);
      }
    }
  }
  if (warp == 1) {
    tmem_alloc(&s.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int j = kStages; j < ntiles; ++j) {  // the first kStages tiles were requested before the set-up barrier
        const int st = j % kStages;
        if (!mbar_wait_for(a.wait_cycles, &s.kv_empty[st], ((j / kStages) & 1) ^ 1)) {
          atomicCAS(a.status, 0u, 101u);
          break;
        }
        mbar_expect_tx(&s.kv_full[st], (kHasT ? 4 : 2) * kBN * D * 2);
        for (int x = 0; x < kBoxes; ++x) {
          tma_load_4d(s.kv[st][0][x], &maps.k, &s.kv_full[st], 64 * x, j * kBN, h, b);
          if (kHasT) tma_load_4d(s.kv[st][1][x], &maps.tk, &s.kv_full[st], 64 * x, j * kBN, h, b);
          tma_load_4d(s.kv[st][2][x], &maps.v, &s.kv_full[st], 64 * x, j * kBN, h, b);
          if (kHasT) tma_load_4d(s.kv[st][3][x], &maps.tv, &s.kv_full[st], 64 * x, j * kBN, h, b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(kBM, kBN, kBf16, false, false);
      constexpr uint32_t idesc_o = make_idesc(kBM, D, kBf16, false, true);
      // products that share their A operand and have adjacent B tiles / accumulators go out as one instruction of
      // twice the width (fewer instructions for the one issuing thread; N = 128 runs at the full tensor rate)
      constexpr bool kMerge = kBoxes == 1;
      constexpr uint32_t idesc_s2 = make_idesc(kBM, 2 * kBN, kBf16, false, false);
      constexpr uint32_t idesc_o2 = make_idesc(kBM, 2 * D <= 256 ? 2 * D : D, kBf16, false, true);
      const uint32_t base16 = smem_u32(&s) >> 4;
      constexpr uint32_t kQTile = kBM * 128, kKvTile = kBN * 128;  // bytes of one 64-channel box
      bool ok = mbar_wait_for(a.wait_cycles, &s.q_full, 0);
      if (!ok) atomicCAS(a.status, 0u, 102u);
      for (int j = 0; ok && j < ntiles; ++j) {
        const int st = j % kStages;
        if (!mbar_wait_for(a.wait_cycles, &s.kv_full[st], (j / kStages) & 1)) {
          atomicCAS(a.status, 0u, 103u);
          break;
        }
        tc_fence_after();
        // S = Q K^T ; Sd = Qd K^T + Q Kd^T      (K-major operands, 16 channels per instruction; one
        // accumulator at a time).  Descriptors are one runtime base word plus compile-time offsets: this one
        // thread issues every MMA of the CTA, so instructions per MMA bound the tensor throughput.
        const uint32_t kvlo = base16 + (uint32_t)((offsetof(Smem, kv) + (size_t)st * 4 * kBoxes * kKvTile) >> 4);
        auto qd = [&](size_t member, int kk) {
          return base16 + (uint32_t)((member + (kk >> 2) * kQTile + (kk & 3) * 32) >> 4) + kDescLoKMajor;
        };
        auto kd = [&](int t, int kk) {
          return kvlo + (uint32_t)(((t * kBoxes + (kk >> 2)) * kKvTile + (kk & 3) * 32) >> 4) + kDescLoKMajor;
        };
        if (!kHasT) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) mma_ss_lo(tmem + kColS, qd(offsetof(Smem, q), kk), kd(0, kk), idesc_s, kk > 0);
        } else if (kMerge) {
          // [S | Sd] = Q [K ; Kd]^T in one N = 128 instruction per step, then Sd += Qd K^T
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) mma_ss_lo(tmem + kColS, qd(offsetof(Smem, q), kk), kd(0, kk), idesc_s2, kk > 0);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) mma_ss_lo(tmem + kColSd, qd(offsetof(Smem, tq), kk), kd(0, kk), idesc_s, true);
        } else {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) mma_ss_lo(tmem + kColS, qd(offsetof(Smem, q), kk), kd(0, kk), idesc_s, kk > 0);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            mma_ss_lo(tmem + kColSd, qd(offsetof(Smem, tq), kk), kd(0, kk), idesc_s, kk > 0);
            mma_ss_lo(tmem + kColSd, qd(offsetof(Smem, q), kk), kd(1, kk), idesc_s, true);
          }
        }
        tc_commit(&s.s_full);
        if (!mbar_wait_for(a.wait_cycles, &s.p_full, j & 1)) {
          atomicCAS(a.status, 0u, 104u);
          break;
        }
        tc_fence_after();
        // O += P V ; Od' += U V + P Vd          (A from TMEM, B = value tile read MN-major, 16 keys per instruction)
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk) {
          // value tiles read MN-major: 16 keys = 2 KiB per step; consecutive 64-channel column blocks (and, for
          // D = 64, V followed by Vd) are kBN * 128 bytes apart
          const uint32_t dv = kvlo + (uint32_t)((2 * kBoxes * kKvTile + kk * 2048) >> 4) + desc_lo_mn_major(kKvTile);
          const uint32_t dtv = kvlo + (uint32_t)((3 * kBoxes * kKvTile + kk * 2048) >> 4) + desc_lo_mn_major(kKvTile);
          const bool acc = (j > 0) || (kk > 0);
          if (!kHasT) {
            mma_ts_lo(tmem + kColO, tmem + kColS + kk * 8, dv, idesc_o, acc);     // O += P V
          } else if (kMerge) {
            mma_ts_lo(tmem + kColO, tmem + kColS + kk * 8, dv, idesc_o2, acc);    // [O | Od'] += P [V | Vd]
            mma_ts_lo(tmem + kColOd, tmem + kColSd + kk * 8, dv, idesc_o, true);  // Od' += U V
          } else {
            mma_ts_lo(tmem + kColO, tmem + kColS + kk * 8, dv, idesc_o, acc);
            mma_ts_lo(tmem + kColOd, tmem + kColSd + kk * 8, dv, idesc_o, acc);
            mma_ts_lo(tmem + kColOd, tmem + kColS + kk * 8, dtv, idesc_o, true);
          }
        }
        tc_commit(&s.kv_empty[st]);
        tc_commit(&s.o_done);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warps: one thread per query row
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t tlane = tmem + ((uint32_t)(quad * 32) << 16);
    const float sl2 = a.scale * kLog2e;
    float m = -INFINITY, l = 0.f, mu = 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      // tcgen05.ld / st are warp-collective: keep every decision that guards them warp-uniform
      if (!__all_sync(0xffffffffu, mbar_wait_for(a.wait_cycles, &s.s_full, j & 1))) {
        atomicCAS(a.status, 0u, 105u);
        ok = false;
        break;
      }
      tc_fence_after();
      // the 64 scores of this row and the first half of Sd in flight at once, one wait
      uint32_t sv[64], sd[32];
      {
        uint32_t(&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sv[0]);
        uint32_t(&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sv[32]);
        tmem_ld32(tlane + kColS, lo);
        tmem_ld32(tlane + kColS + 32, hi);
        if (kHasT) tmem_ld32(tlane + kColSd, sd);
        tc_wait_ld();
      }
      const int nvalid = a.Lk - j * kBN;  // >= 1; < 64 only on the last tile
      if (nvalid < 64) {
#pragma unroll
        for (int c = 0; c < 64; ++c)
          if (c >= nvalid) sv[c] = __float_as_uint(-INFINITY);
      }
      // row max of the raw scores on four independent chains (scale > 0 commutes with the max)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 64; c += 4) {
#pragma unroll
        for (int t = 0; t < 4; ++t) mx4[t] = fmaxf(mx4[t], __uint_as_float(sv[c + t]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sl2;
      // Keep the old reference max while the new one is within the threshold above it: O / Od' then need no rescale.
      float m_new = (mx - m > RescaleThreshold<T>::value) ? mx : m;
      if (j == 0) m_new = mx;
      const float alpha = fast_exp2(m - m_new);  // 1 when unchanged, 0 on the first tile
      if (j > 0 && __any_sync(0xffffffffu, m_new != m)) {
        // S of this tile is complete, so every earlier O / Od' update has retired: safe to rescale in place.
#pragma unroll
        for (int c = 0; c < (kHasT ? 2 : 1) * D; c += 32) {
          uint32_t r[32];
          tmem_ld32(tlane + kColO + c, r);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(tlane + kColO + c, r);
        }
      }
      m = m_new;
      // p = 2^(s * scale*log2e - m), u = p * scale * sd: packed two-wide fp32 arithmetic, two sum chains each
      const float2 sl2x2 = make_float2(sl2, sl2), negm = make_float2(-m, -m), scx2 = make_float2(a.scale, a.scale);
      float2 psum[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      float2 usum[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t pk[16], uk[16];
        if (kHasT && c0 > 0) {
          tmem_ld32(tlane + kColSd + c0, sd);
          tc_wait_ld();
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 t = __ffma2_rn(make_float2(__uint_as_float(sv[c0 + 2 * i]), __uint_as_float(sv[c0 + 2 * i + 1])), sl2x2, negm);
          const float2 p = make_float2(fast_exp2(t.x), fast_exp2(t.y));
          psum[i & 1] = __fadd2_rn(psum[i & 1], p);
          pk[i] = pack2<T>(p.x, p.y);
          if (kHasT) {
            const float2 u = __fmul2_rn(__fmul2_rn(p, scx2),
                                        make_float2(__uint_as_float(sd[2 * i]), __uint_as_float(sd[2 * i + 1])));
            usum[i & 1] = __fadd2_rn(usum[i & 1], u);
            uk[i] = pack2<T>(u.x, u.y);
          }
        }
        // 32 score columns become 16 packed operand columns, written over columns already consumed
        tmem_st16(tlane + kColS + c0 / 2, pk);
        if (kHasT) tmem_st16(tlane + kColSd + c0 / 2, uk);
      }
      l = l * alpha + ((psum[0].x + psum[0].y) + (psum[1].x + psum[1].y));
      mu = mu * alpha + ((usum[0].x + usum[0].y) + (usum[1].x + usum[1].y));
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&s.p_full);
    }
    // ---- epilogue: O = acc / l ; Od = Od'/l - (mu/l) O ; statistics
    if (ok && !__all_sync(0xffffffffu, mbar_wait_for(a.wait_cycles, &s.o_done, (ntiles - 1) & 1))) {
      atomicCAS(a.status, 0u, 106u);
      ok = false;
    }
    tc_fence_after();
    const int qrow = q0 + row;
    const bool live = qrow < a.Lq;  // rows past len_q are clipped by the TMA store
    if (ok) {
      // Every MMA of this CTA has retired, so the Q / Qd tiles are dead: O and Od are staged over them in the
      // 128-byte-swizzled box layout and leave through TMA stores (coalesced; per-lane global stores are far slower).
      const float inv = 1.f / l;
      const float mun = mu * inv;
#pragma unroll
      for (int c = 0; c < D; c += 32) {
        uint32_t ro[32], rd[32];
        tmem_ld32(tlane + kColO + c, ro);
        if (kHasT) tmem_ld32(tlane + kColOd + c, rd);
        tc_wait_ld();
        unsigned char *otile = reinterpret_cast<unsigned char *>(s.q[c / 64]);
        unsigned char *dtile = reinterpret_cast<unsigned char *>(s.tq[c / 64]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t po[4], pd[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const int e = 8 * i + 2 * t;
            const float o0 = __uint_as_float(ro[e]) * inv, o1 = __uint_as_float(ro[e + 1]) * inv;
            po[t] = pack2<T>(o0, o1);
            if (kHasT)
              pd[t] = pack2<T>(__uint_as_float(rd[e]) * inv - mun * o0, __uint_as_float(rd[e + 1]) * inv - mun * o1);
          }
          const uint32_t off = swizzle128_offset(row, (c % 64) / 8 + i);
          *reinterpret_cast<uint4 *>(otile + off) = make_uint4(po[0], po[1], po[2], po[3]);
          if (kHasT) *reinterpret_cast<uint4 *>(dtile + off) = make_uint4(pd[0], pd[1], pd[2], pd[3]);
        }
      }
      fence_proxy_async();
      if (live) {
        const size_t si = ((size_t)b * a.H + h) * a.stat_len + qrow;
        a.lse[si] = m * kLn2 + __logf(l);
        if (kHasT) a.mu[si] = mun;
        if (a.li) a.li[si] = l;
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");  // all four softmax warps, whether or not their waits succeeded
    if (threadIdx.x == 64 && ok) {
      for (int x = 0; x < kBoxes; ++x) {
        tma_store_4d(&maps.o, s.q[x], 64 * x, q0, h, b);
        if (kHasT) tma_store_4d(&maps.to, s.tq[x], 64 * x, q0, h, b);
      }
      tma_store_commit();
      tma_store_wait_read();  // the tiles must stay until the stores have read them; the writes finish on their own
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

template <int D, typename T, bool kHasT>
cudaError_t launch_fwd(const FwdArgs &a, cudaStream_t stream) {
  FwdMaps maps;
  const View *views[8] = {&a.q, &a.tq, &a.k, &a.tk, &a.v, &a.tv, &a.o, &a.to};
  CUtensorMap *dst[8] = {&maps.q, &maps.tq, &maps.k, &maps.tk, &maps.v, &maps.tv, &maps.o, &maps.to};
  for (int i = 0; i < 8; ++i) {
    if (!kHasT && (i & 1)) continue;  // the tangent-side tensors are absent
    const bool is_q = i < 2 || i >= 6;
    if (!make_tensor_map(dst[i], views[i]->ptr, a.dtype, a.B, a.H, is_q ? a.Lq : a.Lk, D, views[i]->sb, views[i]->sh,
                         views[i]->sl, is_q ? kBM : kBN))
      return cudaErrorInvalidValue;
  }
  auto kernel = sm100_fwd_kernel<D, T, kHasT>;
  const size_t smem = sizeof(FwdSmem<D>) + 1024;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid((a.Lq + kBM - 1) / kBM, a.H, a.B);
  {
    LaunchScope scope(kIdFwdTc, stream);
    kernel<<<grid, kThreads, smem, stream>>>(maps, a);
  }
  return cudaGetLastError();
}

}  // namespace

bool sm100_fwd_supported(const FwdArgs &a) {
  if (a.D != 64 && a.D != 128) return false;
  if (a.Lq < 1 || a.Lk < 1 || a.H > 65535 || a.B > 65535) return false;
  const View *qside[4] = {&a.q, &a.o, &a.tq, &a.to}, *kside[4] = {&a.k, &a.v, &a.tk, &a.tv};
  const int n = a.has_t ? 4 : 2;  // the tangent-side views exist only with tangents
  for (int i = 0; i < n; ++i)
    if (!tma_view_ok(*qside[i], a.B, a.H, a.Lq, a.D) || !tma_view_ok(*kside[i], a.B, a.H, a.Lk, a.D)) return false;
  return true;
}

template <typename T>
cudaError_t dispatch_fwd(const FwdArgs &a, cudaStream_t stream) {
  if (a.has_t) return a.D == 64 ? launch_fwd<64, T, true>(a, stream) : launch_fwd<128, T, true>(a, stream);
  return a.D == 64 ? launch_fwd<64, T, false>(a, stream) : launch_fwd<128, T, false>(a, stream);
}

cudaError_t sm100_fwd(const FwdArgs &a, cudaStream_t stream) {
  return a.dtype == JVPATTN_BF16 ? dispatch_fwd<__nv_bfloat16>(a, stream) : dispatch_fwd<__half>(a, stream);
}

}  // namespace jvpattn
