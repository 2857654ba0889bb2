// Attention-JVP backward for sm_100a: the VJPs of cotangents gO (on O) and G (on Od) with respect to
// q, k, v and their tangents, from the saved row statistics (lse, mu).  tcgen05 MMAs with TMEM
// accumulators, TMA-staged tiles, warp-specialised load / MMA / softmax-algebra roles.
//
// Maths (closed form of what semicat/jvp_utils/flash_jvp_backward.py:87-2290 and
// semicat/jvp_utils/flash_attn_triton.py:406-685 compute), per (batch, head):
//   P  = exp(scale QK^T - lse)            N = scale (Qd K^T + Q Kd^T) - mu
//   A  = G V^T                            C = G Vd^T + gO V^T
//   delta = rowsum(G o O)                 dsum = rowsum(G o Od) + rowsum(gO o O)
//   W1 = scale P o (A - delta)            W2 = scale P o ((A - delta) o N + C - dsum)
//   dQd = W1 K      dQ = W1 Kd + W2 K     dKd = W1^T Q     dK = W1^T Qd + W2^T Q
//   dVd = P^T G     dV = (P o N)^T G + P^T gO
// The reference gets delta / dsum from an extra L^2 pass (flash_jvp_backward.py:2012-2290); here they are
// d-length row dot products computed by a small bandwidth-bound kernel into the caller's workspace.
//
// One kernel template serves both sides.  A CTA owns 128 rows of the "resident" side X and streams tiles of
// the other side Y:
//   query owner   X = (Q, Qd, G, gO)   Y = (K, Kd, V, Vd)     -> dQ, dQd
//   key owner     X = (K, Kd, V, Vd)   Y = (Q, Qd, G, gO)     -> dK, dKd, dV, dVd
// For either owner the score tiles are S = X0 Y0^T, Sd = X1 Y0^T + X0 Y1^T, A = X2 Y2^T, C = X2 Y3^T + X3 Y2^T
// (for the key owner these are the transposes, rows = keys), and the outputs are
//   dX1 = W1 Y0,  dX0 = W1 Y1 + W2 Y0,  and for the key owner dVd = P Y2, dV = (P o N) Y2 + P Y3.
// The 16-bit operands P, PoN, W1, W2 are written over the fp32 score columns in TMEM and fed back to the
// tensor core as the A operand; the Y tiles are read MN-major as the B operand.
//
//   warp 0      TMA producer (X once, Y through a 2-stage ring)
//   warp 1      MMA issuer (query owner: the score products)
//   last warp   query owner only: second MMA issuer (the output products)
//   warps 2..   kParts threads per owned row (each on 1/kParts of the tile's columns): score algebra, operand
//               write-back over consumed score columns, epilogue.  Four threads per row where a tile has 64
//               columns (18 warps): the algebra is a chain of tensor-memory reads, exponentials and tensor-memory
//               writes, and with two warps per scheduler its latency, not its instruction count, set the tile time
#include <algorithm>

#include "jvpattn_common.cuh"
#include "sm100_attn.cuh"
#include "sm100_ptx.cuh"

namespace jvpattn {
namespace {

using namespace ptx;

constexpr int kRows = 128;
// threads of a CTA: TMA warp, MMA warp, 4 * parts score-algebra warps, and the second MMA warp of the query owner
__host__ __device__ constexpr int bwd_threads(int parts) { return 64 + 128 * parts + 32; }
// score-algebra threads per owned row: each handles at least 16 columns of a streamed tile
#ifndef JVPATTN_BWD_PARTS_WIDE
#define JVPATTN_BWD_PARTS_WIDE 2
#endif
__host__ __device__ constexpr int bwd_parts(int tile) { return tile >= 64 ? JVPATTN_BWD_PARTS_WIDE : 2; }

template <int D, int TILE>
struct BwdSmem {
  static constexpr int kBoxes = D / 64;
  static constexpr int kXBuf = D == 64 ? 2 : 1;  // owned-row tiles are double buffered where shared memory allows
  static constexpr int kStages = 2;
  alignas(1024) uint16_t x[kXBuf][4][kBoxes][kRows * 64];
  // streamed tiles, 64-channel box outermost: within a box the four tensors are adjacent, so that [Y0 ; Y1] and
  // [Y2 ; Y3] are each one K-major B operand of 2 TILE rows (merged score products) at any head dimension
  alignas(1024) uint16_t y[kStages][kBoxes][4][TILE * 64];
  float4 stats[2][TILE];  // key owner only: per query column {lse*log2e, mu, delta, dsum} (double buffered)
  // Query owner: the owned rows' statistics {lse, mu, delta, dsum} as four float arrays, brought in by bulk copies
  // that complete on the same barrier as the rows.  Its compute warps then issue no global loads at all: a load in
  // flight holds a scoreboard slot that the tensor-memory reads of the score algebra also wait on, which exposed
  // the memory latency once per item even with nothing depending on the load.
  alignas(16) float xstat[kXBuf][4][kRows];
  uint64_t x_full[kXBuf], x_empty[kXBuf], acc_free, y_full[kStages], y_empty[kStages], s1_full, s2_full, c1_done, c2_done[2], r2_free, done, vdone;
  uint32_t tmem_base;
};


// Number of SMs of the current device (cached per device id).
int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

struct BwdMaps {
  CUtensorMap x[4], y[4];
  CUtensorMap out[4];  // dX0, dX1, dV, dVd as 128-row x 64-channel store boxes (D = 64 only)
};

struct BwdKernelArgs {
  View out[4];            // dX0, dX1, dV, dVd (unused entries have ptr == nullptr)
  const float *lse, *mu;  // [B, H, stat_len]
  const float *delta, *dsum;
  unsigned int *status;
  long long wait_cycles;           // budget of every bounded wait
  int B, H, Lx, Ly, Lq, stat_len;  // Lx rows on the owner side, Ly on the streamed side
  int xmask, ymask;             // which of the four X / Y tensors are loaded
  int has_t, has_o;
  float scale;
};

// rows of (G o O), (G o Od) + (gO o O): D/8 threads per row, 16-byte loads
template <int D, typename T>
__global__ void __launch_bounds__(256) row_dots_kernel(BwdArgs a, float *delta, float *dsum) {
  constexpr int kTpr = D / 8;
  ptx::griddep_launch_dependents();  // the query-owner launch may set up while this kernel drains
  const int64_t nrows = (int64_t)a.B * a.H * a.Lq;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t r = gid / kTpr;
  const int part = (int)(gid % kTpr);
  float d1 = 0.f, d2 = 0.f;
  const bool live = r < nrows;
  int b = 0, h = 0, i = 0;
  if (live) {
    i = (int)(r % a.Lq);
    h = (int)((r / a.Lq) % a.H);
    b = (int)(r / ((int64_t)a.Lq * a.H));
    auto load8 = [&](const View &v, float (&f)[8]) {
      const uint4 u = *reinterpret_cast<const uint4 *>(static_cast<const T *>(v.ptr) + v.offset(b, h, i) + part * 8);
      const T *e = reinterpret_cast<const T *>(&u);
#pragma unroll
      for (int t = 0; t < 8; ++t) f[t] = Elem<T>::to_f(e[t]);
    };
    float o[8], x[8], g[8];
    load8(a.o, o);
    if (a.g_to.ptr) {
      load8(a.g_to, g);
      load8(a.to, x);
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        d1 = fmaf(g[t], o[t], d1);
        d2 = fmaf(g[t], x[t], d2);
      }
    }
    if (a.g_o.ptr) {
      load8(a.g_o, g);
#pragma unroll
      for (int t = 0; t < 8; ++t) d2 = fmaf(g[t], o[t], d2);
    }
  }
#pragma unroll
  for (int off = kTpr / 2; off > 0; off >>= 1) {
    d1 += __shfl_xor_sync(0xffffffffu, d1, off);
    d2 += __shfl_xor_sync(0xffffffffu, d2, off);
  }
  if (live && part == 0) {
    const size_t si = ((size_t)b * a.H + h) * a.stat_len + i;
    delta[si] = d1;
    dsum[si] = d2;
  }
}

template <int D, int TILE, bool kKV, bool kDoK, bool kDoV, typename T>
__global__ void __launch_bounds__(bwd_threads(bwd_parts(TILE))) sm100_bwd_kernel(const __grid_constant__ BwdMaps maps, BwdKernelArgs a) {
  constexpr int kParts = bwd_parts(TILE);
  constexpr int kComputeThreads = 128 * kParts;
  extern __shared__ unsigned char smem_raw[];
  using Smem = BwdSmem<D, TILE>;
  Smem &s = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kBoxes = D / 64;
  constexpr int kStages = Smem::kStages;
  constexpr int kAcc = (kDoK ? 2 : 0) + (kDoV ? 2 : 0);
  // accumulators; the tangent-gradient tile sits below its partner so that one N = 2D instruction can update both
  constexpr uint32_t kColKd = 0, kColK = D;                          // dX1, dX0
  constexpr uint32_t kColVd = kDoK ? 2 * D : 0, kColV = kColVd + D;  // dVd, dV
  // two score regions that are in different phases of the pipeline: (S | Sd) and (A | C)
  constexpr uint32_t kColS = kAcc * D, kColSd = kColS + TILE, kColA = kColS + 2 * TILE, kColC = kColS + 3 * TILE;
  // Query owner: its two accumulators leave room for a separate, double-buffered home of the W1 / W2 operands
  // (TILE / 2 packed columns each), so that the (A | C) region is free again as soon as the score algebra has read it
  // instead of when the output products have consumed the operands written over it.
  constexpr bool kSplit = !kKV;
  constexpr uint32_t kColW = kAcc * D + 4 * TILE;
  constexpr uint32_t kUsed = kColW + (kSplit ? 2 * TILE : 0);
  static_assert(kUsed <= 512, "TMEM budget");
  constexpr uint32_t kTmemCols = kUsed <= 256 ? 256 : 512;
  constexpr bool kBf16 = IsBf16<T>::value;
  constexpr uint32_t kTileBytes = TILE * D * 2;
  constexpr int CH = TILE / kParts;  // score columns per compute thread and tile
  static_assert(CH % 16 == 0, "a compute thread reads its score columns 16 at a time");
  // d = 64 key owner: dV / dVd are final one group before dK / dKd (their last products are issued ahead of the last
  // tile's second half), so they are staged for the output stores while the tensor core finishes dK / dKd
  constexpr bool kEarlyV = kKV && kDoK && kDoV && kBoxes == 1;

  constexpr int kXBuf = Smem::kXBuf;
  constexpr int kWarpB = 2 + 4 * kParts;  // the second MMA issuer sits behind the score-algebra warps
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntiles = (a.Ly + TILE - 1) / TILE;
  const bool has_t = a.has_t != 0, has_o = a.has_o != 0;
  // Persistent CTA: work item = 128 owned rows of one (batch, head); items blockIdx.x, + gridDim.x, ...
  // Counters shared by all roles: n = items done by this CTA, g = streamed tiles done (across items).
  const int nx = (a.Lx + kRows - 1) / kRows;
  const int items = a.B * a.H * nx;
  auto decode = [&](int it, int &bb, int &hh, int &xx0) {
    // Short sequences (a step's tensors are a few L2 sizes): the query owner walks the items from the back, the key
    // owner from the front, so that each launch starts with the (batch, head) pairs that the launch before it (the
    // forward front to back, then the query owner back to front) touched last, while their tensors are still in L2.
    // At long sequences a launch outlives the cache many times over and the order is the plain one.
    if (!kKV && ntiles <= 8) it = items - 1 - it;
    xx0 = (it % nx) * kRows;
    const int bh = it / nx;
    hh = bh % a.H;
    bb = bh / a.H;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < kXBuf; ++i) {
      mbar_init(&s.x_full[i], 1);
      mbar_init(&s.x_empty[i], kBoxes == 1 ? 2 : 1);  // MMA issuer, plus the thread whose output stores read the buffer
    }
    mbar_init(&s.acc_free, kComputeThreads);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&s.y_full[i], 1);
      mbar_init(&s.y_empty[i], 1);
    }
    mbar_init(&s.s1_full, 1);
    mbar_init(&s.s2_full, 1);
    mbar_init(&s.c1_done, kComputeThreads);
    mbar_init(&s.c2_done[0], kComputeThreads);
    mbar_init(&s.c2_done[1], kComputeThreads);
    mbar_init(&s.r2_free, kComputeThreads);
    mbar_init(&s.done, 1);
    mbar_init(&s.vdone, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&s.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s.tmem_base;
  // Launch overlap (programmatic dependent launch).  The row-dot kernel is launched normally, so everything earlier
  // in the stream has completed when it runs, and it releases its dependents at once.  The query owner, launched
  // with the programmatic-serialization attribute, sets up and requests its first row tiles while the row-dot
  // kernel drains; only its producer thread reads what that kernel wrote (delta, dsum), so that thread alone
  // waits for it, and it releases the key-owner launches right after.  Those read nothing the query owner writes:
  // their CTAs move onto SMs as query-owner CTAs leave, which hides their start-up and fills the tail in which
  // only some SMs still hold a query-owner item.  A key-owner CTA can only exist after every query-owner producer
  // has passed its wait, hence after the row dots are complete.
  if (kKV) griddep_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&maps.x[0]);
      prefetch_tensormap(&maps.y[0]);
      int n = 0, g = 0;
      bool ok = true;
      // owned-row tiles of work item `it_` (the n_-th of this CTA) into X buffer n_ % kXBuf
      auto load_x = [&](int it_, int n_) -> bool {
        int b, h, x0;
        decode(it_, b, h, x0);
        const int xb = n_ % kXBuf;
        if (!mbar_wait_for(a.wait_cycles, &s.x_empty[xb], ((n_ / kXBuf) & 1) ^ 1)) {
          atomicCAS(a.status, 0u, 209u);
          return false;
        }
        mbar_expect_tx(&s.x_full[xb], __popc(a.xmask) * kRows * D * 2 + (kKV ? 0 : (has_t ? 4 : 3) * kRows * 4));
        for (int t = 0; t < 4; ++t)
          if (a.xmask >> t & 1)
            for (int x = 0; x < kBoxes; ++x) tma_load_4d(s.x[xb][t][x], &maps.x[t], &s.x_full[xb], 64 * x, x0, h, b);
        if (!kKV) {
          if (n_ == 0) griddep_wait();  // delta / dsum are the row-dot kernel's output
          const size_t si = ((size_t)b * a.H + h) * a.stat_len + x0;  // stat_len is a multiple of 128: always in bounds
          bulk_load_1d(s.xstat[xb][0], a.lse + si, kRows * 4, &s.x_full[xb]);
          if (has_t) bulk_load_1d(s.xstat[xb][1], a.mu + si, kRows * 4, &s.x_full[xb]);
          bulk_load_1d(s.xstat[xb][2], a.delta + si, kRows * 4, &s.x_full[xb]);
          bulk_load_1d(s.xstat[xb][3], a.dsum + si, kRows * 4, &s.x_full[xb]);
          if (n_ == 0) griddep_launch_dependents();
        }
        if (kXBuf == 1 && it_ + (int)gridDim.x < items) {  // single X buffer: at least bring the next item's rows into L2
          decode(it_ + gridDim.x, b, h, x0);
          for (int t = 0; t < 4; ++t)
            if (a.xmask >> t & 1)
              for (int x = 0; x < kBoxes; ++x) tma_prefetch_4d(&maps.x[t], 64 * x, x0, h, b);
        }
        return true;
      };
      // A streamed tile can only be requested once its stage is free, one tile ahead at best, which is less
      // than the DRAM latency when an item has few tiles: the tile `kAhead` positions further down this CTA's
      // stream is therefore pulled into L2 when a tile is requested.
      constexpr int kAhead = 2;
      auto prefetch_y = [&](int n_, int j_) {
        const int pos = j_ + kAhead;
        const int it_ = blockIdx.x + (n_ + pos / ntiles) * (int)gridDim.x;
        if (it_ >= items) return;
        int b, h, x0;
        decode(it_, b, h, x0);
        for (int t = 0; t < 4; ++t)
          if (a.ymask >> t & 1)
            for (int x = 0; x < kBoxes; ++x) tma_prefetch_4d(&maps.y[t], 64 * x, (pos % ntiles) * TILE, h, b);
      };
      // With two X buffers the next item's rows are requested as soon as this item's first two streamed tiles
      // are on their way, so they are resident long before the item starts.
      const int jx = kXBuf == 2 ? (ntiles < 2 ? ntiles - 1 : 1) : -1;
      if (blockIdx.x < items) ok = load_x(blockIdx.x, 0);
      for (int it = blockIdx.x; ok && it < items; it += gridDim.x, ++n) {
        int b, h, x0;
        decode(it, b, h, x0);
        if (kXBuf == 1 && n > 0 && !(ok = load_x(it, n))) break;
        for (int j = 0; j < ntiles; ++j, ++g) {
          const int st = g % kStages;
          if (!mbar_wait_for(a.wait_cycles, &s.y_empty[st], ((g / kStages) & 1) ^ 1)) {
            atomicCAS(a.status, 0u, 201u);
            ok = false;
            break;
          }
          mbar_expect_tx(&s.y_full[st], __popc(a.ymask) * kTileBytes);
          for (int t = 0; t < 4; ++t)
            if (a.ymask >> t & 1)
              for (int x = 0; x < kBoxes; ++x) tma_load_4d(s.y[st][x][t], &maps.y[t], &s.y_full[st], 64 * x, j * TILE, h, b);
          prefetch_y(n, j);
          if (j == jx && it + (int)gridDim.x < items && !(ok = load_x(it + gridDim.x, n + 1))) break;
        }
      }
    }
  } else if (warp == 1 || warp == kWarpB) {
    // ------------------------------------------------------------------ MMA issuer
    // Per streamed tile j the tensor core runs four groups, interleaved with the two halves of the score
    // algebra so that it always has the next group queued while the compute warps work:
    //   scores1(j): S, Sd            -> compute1(j): P, PoN (operands), keeps scale*P and N in registers
    //   scores2(j): A, C             -> compute2(j): W1, W2 (operands)
    //   outV(j):    dVd, dV += ...   needs compute1(j)         outK(j): dX1, dX0 += ...   needs compute2(j)
    // issue order: scores1(0) scores2(0) | outV(j) scores1(j+1) outK(j) scores2(j+1) | ...
    if (lane == 0 && (warp == 1 || kSplit)) {
      constexpr uint32_t idesc_s = make_idesc(kRows, TILE, kBf16, false, false);
      constexpr uint32_t idesc_o = make_idesc(kRows, D, kBf16, false, true);
      // Pairs of products that share their A operand and whose B tiles / accumulators are adjacent are issued as
      // one instruction of twice the width: fewer instructions for the single issuing thread, and N = 128
      // instructions run at the full tensor rate where N = 64 ones reach about two thirds of it.
      constexpr bool kMergeS = 2 * TILE <= 256;                   // score products: [S | Sd], [A | C]
      constexpr bool kMerge = (kBoxes == 1) && (2 * D <= 256);    // output products: [dX1 | dX0], [dVd | dV]
      constexpr uint32_t idesc_s2 = make_idesc(kRows, 2 * TILE, kBf16, false, false);
      constexpr uint32_t idesc_o2 = make_idesc(kRows, 2 * D, kBf16, false, true);
      // the X2 Y3^T term of C carries G Vd^T for the query owner but V gO^T for the key owner, and vice versa
      const bool term23 = kKV ? has_o : has_t;
      const bool term32 = kKV ? has_t : has_o;
      // Low descriptor words: one runtime base (shared memory offset >> 4) plus compile-time tile offsets, so
      // that issuing an MMA costs a handful of instructions (the issue rate of this one thread bounds the kernel).
      const uint32_t base16 = smem_u32(&s) >> 4;
      constexpr uint32_t kXTile = kRows * 128, kYTile = TILE * 128;  // bytes of one 64-channel box
      auto xbase = [&](int xb) { return base16 + (uint32_t)((offsetof(Smem, x) + (size_t)xb * 4 * kBoxes * kXTile) >> 4); };
      auto ybase = [&](int st) { return base16 + (uint32_t)((offsetof(Smem, y) + (size_t)st * 4 * kBoxes * kYTile) >> 4); };
      auto xd = [&](uint32_t xlo, int t, int kk) {
        return xlo + (uint32_t)(((t * kBoxes + (kk >> 2)) * kXTile + (kk & 3) * 32) >> 4) + kDescLoKMajor;
      };
      auto yd = [&](uint32_t ylo, int t, int kk) {
        return ylo + (uint32_t)((((kk >> 2) * 4 + t) * kYTile + (kk & 3) * 32) >> 4) + kDescLoKMajor;
      };
      // one accumulator at a time, 16 channels per instruction.  g = tile counter (stage / parity), xb = X buffer,
      // last = this is the item's last tile (its X tiles are released once no later score MMA needs them)
      auto scores1 = [&](int g, int xb, bool last) -> bool {
        const int st = g % kStages;
        if (!mbar_wait_for(a.wait_cycles, &s.y_full[st], (g / kStages) & 1)) return false;
        tc_fence_after();
        const uint32_t xlo = xbase(xb), ylo = ybase(st);
        if (kMergeS && has_t) {
          // [S | Sd] = X0 [Y0 ; Y1]^T in one N = 2 TILE instruction per step, then Sd += X1 Y0^T
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) mma_ss_lo(tmem + kColS, xd(xlo, 0, kk), yd(ylo, 0, kk), idesc_s2, kk > 0);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) mma_ss_lo(tmem + kColSd, xd(xlo, 1, kk), yd(ylo, 0, kk), idesc_s, true);
        } else {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) mma_ss_lo(tmem + kColS, xd(xlo, 0, kk), yd(ylo, 0, kk), idesc_s, kk > 0);
          if (has_t) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              mma_ss_lo(tmem + kColSd, xd(xlo, 1, kk), yd(ylo, 0, kk), idesc_s, kk > 0);
              mma_ss_lo(tmem + kColSd, xd(xlo, 0, kk), yd(ylo, 1, kk), idesc_s, true);
            }
          }
        }
        tc_commit(&s.s1_full);
        if (!kDoK && last) tc_commit(&s.x_empty[xb]);
        return true;
      };
      auto scores2 = [&](int g, int xb, bool last) {
        if (!kDoK) return;
        const int st = g % kStages;  // already resident: scores1 waited for it
        const uint32_t xlo = xbase(xb), ylo = ybase(st);
        bool c_started = false;
        if (kMergeS && has_t && term23) {
          // [A | C] = X2 [Y2 ; Y3]^T in one N = 2 TILE instruction per step
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) mma_ss_lo(tmem + kColA, xd(xlo, 2, kk), yd(ylo, 2, kk), idesc_s2, kk > 0);
          c_started = true;
        } else if (has_t) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) mma_ss_lo(tmem + kColA, xd(xlo, 2, kk), yd(ylo, 2, kk), idesc_s, kk > 0);
        }
        if (term23 && !c_started) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            mma_ss_lo(tmem + kColC, xd(xlo, 2, kk), yd(ylo, 3, kk), idesc_s, c_started || kk > 0);
          c_started = true;
        }
        if (term32) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            mma_ss_lo(tmem + kColC, xd(xlo, 3, kk), yd(ylo, 2, kk), idesc_s, c_started || kk > 0);
        }
        tc_commit(&s.s2_full);
        if (last) tc_commit(&s.x_empty[xb]);
      };
      // Y tiles as MN-major B operands of the output products: consecutive 64-channel blocks are the two boxes of
      // one tensor (d = 128: four tiles apart) or, for the merged d = 64 products, two adjacent tensors
      constexpr uint32_t lbo = (kBoxes == 1 ? 1 : 4) * TILE * 128;
      auto yb = [&](uint32_t ylo, int t, int kk) {
        return ylo + (uint32_t)((t * kYTile + kk * 2048) >> 4) + desc_lo_mn_major(lbo);
      };
      // the thread that owned score columns [16 kk, 16 kk + 16) left its 8 packed operand columns at the start
      // of its own column range (see the score-algebra warps)
      auto oa = [&](int kk) -> uint32_t { return ((16 * kk) / CH) * CH + ((16 * kk) % CH) / 2; };
      if constexpr (kSplit) {
        // ---- query owner: two issuers and a chain-free schedule.
        // Measured per 64-key tile with one issuer: the score algebra needed ~1570 cycles, the tensor pipe ~1280, but a
        // tile took ~3280, because (A | C) of the next tile could only be issued behind the output products of this
        // one (which read W1 / W2 from that region), and those wait for the second half of the score algebra: a serial
        // chain of algebra -> 8 MMAs -> 8 MMAs -> algebra, with every tcgen05.commit on the way holding back its
        // thread's later MMAs until the earlier ones have drained.  Here W1 / W2 have a home of their own, so
        //   issuer A (warp 1):    scores1(j+1) once compute1(j) has read (S | Sd); scores2(j+1) once compute2(j) has
        //                         read (A | C) - neither waits for an output product;
        //   issuer B (last warp): outK(j) once compute2(j) has written W1 / W2; its commits (stage free, item done)
        //                         drain only its own queue.
        // Hazards: W[g & 1] is rewritten by compute2(g + 2), which needs scores2(g + 2), which needs the streamed
        // stage of tile g reloaded, which needs outK(g) complete (y_empty): outK(g) has long read it.
        int it = blockIdx.x, j = 0, n = 0, g = 0;
        bool ok = it < items;
        if (warp == 1) {
          if (ok && !mbar_wait_for(a.wait_cycles, &s.x_full[0], 0)) {
            atomicCAS(a.status, 0u, 202u);
            ok = false;
          }
          if (ok) {
            if (!scores1(0, 0, false)) {
              atomicCAS(a.status, 0u, 203u);
              ok = false;
            } else {
              scores2(0, 0, ntiles == 1);
            }
          }
          while (ok) {
            int it2 = it, j2 = j + 1, n2 = n;
            if (j2 == ntiles) {
              it2 = it + gridDim.x;
              j2 = 0;
              n2 = n + 1;
            }
            if (it2 >= items) break;
            if (!mbar_wait_for(a.wait_cycles, &s.c1_done, g & 1)) {  // (S | Sd) of tile g has been read
              atomicCAS(a.status, 0u, 204u);
              break;
            }
            if (j2 == 0 && !mbar_wait_for(a.wait_cycles, &s.x_full[n2 % kXBuf], (n2 / kXBuf) & 1)) {
              atomicCAS(a.status, 0u, 202u);
              break;
            }
            if (!scores1(g + 1, n2 % kXBuf, false)) {
              atomicCAS(a.status, 0u, 203u);
              break;
            }
            if (!mbar_wait_for(a.wait_cycles, &s.r2_free, g & 1)) {  // (A | C) of tile g has been read
              atomicCAS(a.status, 0u, 215u);
              break;
            }
            tc_fence_after();
            scores2(g + 1, n2 % kXBuf, j2 == ntiles - 1);
            it = it2; j = j2; n = n2; ++g;
          }
        } else {
          const bool acc_merge = kMerge && has_t;
          for (; ok; ) {
            const int st = g % kStages;
            // Two barriers, by tile parity.  Nothing that this thread issues gates the second half of the score algebra,
            // so the compute warps can complete two tiles (g and g + 1) while this thread is still held up behind the
            // other issuer's MMAs, and a parity wait on a single barrier would then take the incomplete phase g + 2
            // for phase g and never return.  Tile g + 2 cannot complete before outK(g) (its streamed stage is reloaded
            // only then), so with one barrier per parity the wait is unambiguous.
            if (!mbar_wait_for(a.wait_cycles, &s.c2_done[g & 1], (g >> 1) & 1)) {  // W1 / W2 of tile g are in place
              atomicCAS(a.status, 0u, 216u);
              break;
            }
            if (j == 0 && !mbar_wait_for(a.wait_cycles, &s.acc_free, (n & 1) ^ 1)) {  // previous item's accumulators have been read out
              atomicCAS(a.status, 0u, 210u);
              break;
            }
            tc_fence_after();
            const uint32_t ylo_out = ybase(st);
            const uint32_t w1 = tmem + kColW + (uint32_t)(g & 1) * TILE, w2 = w1 + TILE / 2;
            if (acc_merge) {
              const bool acc = j > 0;
#pragma unroll
              for (int kk = 0; kk < TILE / 16; ++kk) {
                mma_ts_lo(tmem + kColKd, w1 + 8 * kk, yb(ylo_out, 0, kk), idesc_o2, acc || kk > 0);  // [dX1 | dX0] += W1 [Y0 | Y1]
                mma_ts_lo(tmem + kColK, w2 + 8 * kk, yb(ylo_out, 0, kk), idesc_o, true);          // dX0 += W2 Y0
              }
            } else {
#pragma unroll
              for (int kk = 0; kk < TILE / 16; ++kk) {
                bool init0 = j > 0 || kk > 0;
                if (has_t) {
                  mma_ts_lo(tmem + kColKd, w1 + 8 * kk, yb(ylo_out, 0, kk), idesc_o, init0);   // dX1 += W1 Y0
                  mma_ts_lo(tmem + kColK, w1 + 8 * kk, yb(ylo_out, 1, kk), idesc_o, init0);    // dX0 += W1 Y1
                  init0 = true;
                }
                mma_ts_lo(tmem + kColK, w2 + 8 * kk, yb(ylo_out, 0, kk), idesc_o, init0);      // dX0 += W2 Y0
              }
            }
            tc_commit(&s.y_empty[st]);
            if (j == ntiles - 1) tc_commit(&s.done);
            if (++j == ntiles) {
              it += gridDim.x;
              j = 0;
              ++n;
            }
            ++g;
            if (it >= items) break;
          }
        }
      } else {
      // the stream of (item, tile) pairs this CTA walks; `n` counts items, `g` tiles
      int it = blockIdx.x, j = 0, n = 0, g = 0;
      bool ok = it < items;
      if (ok && !mbar_wait_for(a.wait_cycles, &s.x_full[0], 0)) {
        atomicCAS(a.status, 0u, 202u);
        ok = false;
      }
      if (ok) {
        if (!scores1(0, 0, ntiles == 1)) {
          atomicCAS(a.status, 0u, 203u);
          ok = false;
        } else {
          scores2(0, 0, ntiles == 1);
        }
      }
      bool init0 = false, init1 = false, initv = false, initvd = false;  // accumulators written in this item
      while (ok) {
        const int st = g % kStages;
        // successor in the stream
        int it2 = it, j2 = j + 1, n2 = n;
        if (j2 == ntiles) {
          it2 = it + gridDim.x;
          j2 = 0;
          n2 = n + 1;
        }
        const bool has_next = it2 < items;
        if (j == 0) init0 = init1 = initv = initvd = false;
        if (!mbar_wait_for(a.wait_cycles, &s.c1_done, g & 1)) {
          atomicCAS(a.status, 0u, 204u);
          break;
        }
        if (j == 0 && !mbar_wait_for(a.wait_cycles, &s.acc_free, (n & 1) ^ 1)) {  // previous item's accumulators have been read out
          atomicCAS(a.status, 0u, 210u);
          break;
        }
        tc_fence_after();
        const uint32_t ylo_out = ybase(st);
        // (the common case, both cotangents present, is issued as straight-line code: a run-time condition between
        //  two instructions of a group costs this thread tens of cycles per instruction)
        if (kDoV && kMerge && has_t && has_o) {
          const bool acc = j > 0;
#pragma unroll
          for (int kk = 0; kk < TILE / 16; ++kk) {
            mma_ts_lo(tmem + kColVd, tmem + kColS + oa(kk), yb(ylo_out, 2, kk), idesc_o2, acc || kk > 0);  // [dVd | dV] += P [G | gO]
            mma_ts_lo(tmem + kColV, tmem + kColSd + oa(kk), yb(ylo_out, 2, kk), idesc_o, true);          // dV += (P o N) G
          }
          initv = initvd = true;
        } else if (kDoV) {
#pragma unroll
          for (int kk = 0; kk < TILE / 16; ++kk) {
            if (kMerge && has_t && has_o) {
              mma_ts_lo(tmem + kColVd, tmem + kColS + oa(kk), yb(ylo_out, 2, kk), idesc_o2, initvd);  // [dVd | dV] += P [G | gO]
              mma_ts_lo(tmem + kColV, tmem + kColSd + oa(kk), yb(ylo_out, 2, kk), idesc_o, true);     // dV += (P o N) G
              initv = initvd = true;
            } else {
              if (has_t) {
                mma_ts_lo(tmem + kColVd, tmem + kColS + oa(kk), yb(ylo_out, 2, kk), idesc_o, initvd);  // dVd += P G
                mma_ts_lo(tmem + kColV, tmem + kColSd + oa(kk), yb(ylo_out, 2, kk), idesc_o, initv);   // dV  += (P o N) G
                initv = initvd = true;
              }
              if (has_o) {
                mma_ts_lo(tmem + kColV, tmem + kColS + oa(kk), yb(ylo_out, 3, kk), idesc_o, initv);    // dV  += P gO
                initv = true;
              }
            }
          }
        }
        if (kEarlyV && j == ntiles - 1) tc_commit(&s.vdone);  // dV / dVd of this item are final
        if (has_next) {
          if (j2 == 0 && !mbar_wait_for(a.wait_cycles, &s.x_full[n2 % kXBuf], (n2 / kXBuf) & 1)) {
            atomicCAS(a.status, 0u, 202u);
            break;
          }
          if (!scores1(g + 1, n2 % kXBuf, j2 == ntiles - 1)) {
            atomicCAS(a.status, 0u, 203u);
            break;
          }
        }
        if (kDoK) {
          if (!mbar_wait_for(a.wait_cycles, &s.c2_done[0], g & 1)) {
            atomicCAS(a.status, 0u, 207u);
            break;
          }
          tc_fence_after();
          if (kMerge && has_t) {
            const bool acc = j > 0;
#pragma unroll
            for (int kk = 0; kk < TILE / 16; ++kk) {
              mma_ts_lo(tmem + kColKd, tmem + kColA + oa(kk), yb(ylo_out, 0, kk), idesc_o2, acc || kk > 0);  // [dX1 | dX0] += W1 [Y0 | Y1]
              mma_ts_lo(tmem + kColK, tmem + kColC + oa(kk), yb(ylo_out, 0, kk), idesc_o, true);          // dX0 += W2 Y0
            }
            init0 = init1 = true;
          } else
#pragma unroll
          for (int kk = 0; kk < TILE / 16; ++kk) {
            if (kMerge && has_t) {
              mma_ts_lo(tmem + kColKd, tmem + kColA + oa(kk), yb(ylo_out, 0, kk), idesc_o2, init1);  // [dX1 | dX0] += W1 [Y0 | Y1]
              init0 = init1 = true;
            } else if (has_t) {
              mma_ts_lo(tmem + kColKd, tmem + kColA + oa(kk), yb(ylo_out, 0, kk), idesc_o, init1);   // dX1 += W1 Y0
              mma_ts_lo(tmem + kColK, tmem + kColA + oa(kk), yb(ylo_out, 1, kk), idesc_o, init0);    // dX0 += W1 Y1
              init0 = init1 = true;
            }
            mma_ts_lo(tmem + kColK, tmem + kColC + oa(kk), yb(ylo_out, 0, kk), idesc_o, init0);      // dX0 += W2 Y0
            init0 = true;
          }
        }
        tc_commit(&s.y_empty[st]);
        if (j == ntiles - 1) tc_commit(&s.done);
        if (!has_next) break;
        scores2(g + 1, n2 % kXBuf, j2 == ntiles - 1);
        it = it2; j = j2; n = n2; ++g;
      }
      }  // single issuer
    }
  } else {
    // ------------------------------------------------------------------ score algebra: two threads per owned row
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const int col0 = part * CH;
    const int ctid = threadIdx.x - 64;  // 0..255 among the compute threads
    const uint32_t tlane = tmem + ((uint32_t)(quad * 32) << 16);
    const float sl2 = a.scale * kLog2e;
    const float2 sl2x2 = make_float2(sl2, sl2), scx2 = make_float2(a.scale, a.scale);
    // per-column statistics of the key owner: the first TILE compute threads fetch one query column each,
    // one tile ahead (also across items), and publish it through shared memory
    auto fetch_stat = [&](int it_, int j_) -> float4 {
      int bb, hh, xx;
      decode(it_, bb, hh, xx);
      const int col = j_ * TILE + ctid;
      if (ctid >= TILE || col >= a.Lq) return make_float4(INFINITY, 0.f, 0.f, 0.f);  // padded query: P = 0
      const size_t si = ((size_t)bb * a.H + hh) * a.stat_len + col;
      // raw values: nothing may depend on these loads until they are published a tile later (a dependent
      // instruction here would stall the warp, and with it the barrier below, for the full memory latency)
      return make_float4(a.lse[si], has_t ? a.mu[si] : 0.f, a.delta[si], a.dsum[si]);
    };
    float4 pre = make_float4(0.f, 0.f, 0.f, 0.f);
    if (kKV && blockIdx.x < items) pre = fetch_stat(blockIdx.x, 0);
    bool ok = true;
    int n = 0, g = 0;
    int pending_xb = -1;  // compute thread 0: X buffer whose output stores have been issued but not yet released
   for (int it = blockIdx.x; it < items; it += gridDim.x, ++n) {
    int b, h, x0;
    decode(it, b, h, x0);
    // query owner: this thread's row statistics {lse * log2e, mu, delta, dsum}, delivered with the item's rows
    float4 rstat = make_float4(INFINITY, 0.f, 0.f, 0.f);  // row past the end: P = 0
    if (!kKV) {
      const int xb_ = n % kXBuf;
      if (ok && !__all_sync(0xffffffffu, mbar_wait_for(a.wait_cycles, &s.x_full[xb_], (n / kXBuf) & 1))) {
        atomicCAS(a.status, 0u, 211u);
        ok = false;
      }
      if (ok && x0 + row < a.Lx)
        rstat = make_float4(s.xstat[xb_][0][row] * kLog2e, has_t ? s.xstat[xb_][1][row] : 0.f, s.xstat[xb_][2][row],
                            s.xstat[xb_][3][row]);
    }
    for (int j = 0; j < ntiles; ++j, ++g) {
      if (kKV) {
        if (ctid < TILE) s.stats[g & 1][ctid] = make_float4(pre.x * kLog2e, pre.y, pre.z, pre.w);
        if (j + 1 < ntiles) pre = fetch_stat(it, j + 1);
        else if (it + (int)gridDim.x < items) pre = fetch_stat(it + gridDim.x, 0);
        asm volatile("bar.sync 1, %0;" ::"n"(kComputeThreads) : "memory");
      }
      // a warp whose wait ran out keeps walking the loops without touching TMEM so that the barrier above still matches
      if (ok && !__all_sync(0xffffffffu, mbar_wait_for(a.wait_cycles, &s.s1_full, g & 1))) {
        atomicCAS(a.status, 0u, 205u);
        ok = false;
      }
      if (!ok) continue;
      tc_fence_after();
      const float4 *st = s.stats[g & 1];
      const int nvalid = a.Ly - j * TILE;  // streamed rows in this tile (masking for the query owner)
      // ---- first half: P = exp2(s*scale*log2e - lse*log2e), N = scale*sd - mu
      float2 sp[CH / 2], nn[CH / 2];  // scale * P and N, carried into the second half
#pragma unroll
      for (int c = 0; c < CH; c += 16) {
        const int cs = col0 + c;  // first score column of this chunk
        uint32_t rs[16], rd[16];
        tmem_ld16(tlane + kColS + cs, rs);
        if (has_t) tmem_ld16(tlane + kColSd + cs, rd);
        tc_wait_ld();
        if (!kDoV && c + 16 >= CH) {
          // nothing is written back over the scores: the region is free once this thread's last read has landed
          tc_fence_before();
          mbar_arrive(&s.c1_done);
        }
        if (!kKV && nvalid < TILE) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (cs + i >= nvalid) rs[i] = __float_as_uint(-INFINITY);  // key past the end: P = 0
        }
        uint32_t kp[8], kpn[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 s0 = kKV ? st[cs + 2 * i] : rstat, s1 = kKV ? st[cs + 2 * i + 1] : rstat;
          const float2 t = __ffma2_rn(make_float2(__uint_as_float(rs[2 * i]), __uint_as_float(rs[2 * i + 1])), sl2x2,
                                      make_float2(-s0.x, -s1.x));
          const float2 p = make_float2(fast_exp2(t.x), fast_exp2(t.y));
          float2 n = make_float2(0.f, 0.f);
          if (has_t)
            n = __ffma2_rn(make_float2(__uint_as_float(rd[2 * i]), __uint_as_float(rd[2 * i + 1])), scx2,
                           make_float2(-s0.y, -s1.y));
          sp[c / 2 + i] = __fmul2_rn(p, scx2);
          nn[c / 2 + i] = n;
          if (kDoV) {
            kp[i] = pack2<T>(p.x, p.y);
            if (has_t) {
              const float2 pn = __fmul2_rn(p, n);
              kpn[i] = pack2<T>(pn.x, pn.y);
            }
          }
        }
        if (kDoV) {
          // 16 score columns become 8 packed operand columns, written at the start of this thread's own
          // column range, over columns it has already consumed
          tmem_st8(tlane + kColS + col0 + c / 2, kp);
          if (has_t) tmem_st8(tlane + kColSd + col0 + c / 2, kpn);
        }
      }
      if (kDoV) {
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(&s.c1_done);  // S / Sd consumed (the region may be refilled) and P / PoN in place
      }
      if (pending_xb >= 0) {
        // the previous item's output stores have long finished reading its X buffer: hand it back to the producer
        tma_store_wait_read();
        mbar_arrive(&s.x_empty[pending_xb]);
        pending_xb = -1;
      }
      if (!kDoK) continue;
      // ---- second half: W1 = scale P (A - delta), W2 = scale P ((A - delta) N + C - dsum)
      if (!__all_sync(0xffffffffu, mbar_wait_for(a.wait_cycles, &s.s2_full, g & 1))) {
        atomicCAS(a.status, 0u, 208u);
        ok = false;
        continue;
      }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < CH; c += 16) {
        const int cs = col0 + c;
        uint32_t ra[16], rc[16];
        if (has_t) tmem_ld16(tlane + kColA + cs, ra);
        tmem_ld16(tlane + kColC + cs, rc);
        tc_wait_ld();
        if (kSplit && c + 16 >= CH) {
          tc_fence_before();
          mbar_arrive(&s.r2_free);  // (A | C) read: the next tile's products may overwrite the region
        }
        uint32_t kw1[8], kw2[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 s0 = kKV ? st[cs + 2 * i] : rstat, s1 = kKV ? st[cs + 2 * i + 1] : rstat;
          float2 inner = __fadd2_rn(make_float2(__uint_as_float(rc[2 * i]), __uint_as_float(rc[2 * i + 1])),
                                    make_float2(-s0.w, -s1.w));
          if (has_t) {
            const float2 da = __fadd2_rn(make_float2(__uint_as_float(ra[2 * i]), __uint_as_float(ra[2 * i + 1])),
                                         make_float2(-s0.z, -s1.z));
            const float2 w1 = __fmul2_rn(sp[c / 2 + i], da);
            kw1[i] = pack2<T>(w1.x, w1.y);
            inner = __ffma2_rn(da, nn[c / 2 + i], inner);
          }
          const float2 w2 = __fmul2_rn(sp[c / 2 + i], inner);
          kw2[i] = pack2<T>(w2.x, w2.y);
        }
        if (kSplit) {
          // contiguous packing in the operands' own buffer: key column k of the tile sits in packed column k / 2
          const uint32_t wbase = tlane + kColW + (uint32_t)(g & 1) * TILE + (col0 + c) / 2;
          if (has_t) tmem_st8(wbase, kw1);
          tmem_st8(wbase + TILE / 2, kw2);
        } else {
          if (has_t) tmem_st8(tlane + kColA + col0 + c / 2, kw1);
          tmem_st8(tlane + kColC + col0 + c / 2, kw2);
        }
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&s.c2_done[kSplit ? (g & 1) : 0]);
    }
    // ---- epilogue of the item: accumulators -> 16-bit outputs, each thread 1/kParts of the channels of its row
    {
      const int xr = x0 + row;
      const bool live = xr < a.Lx;
      constexpr int kChan = D / kParts;  // channels per thread
      const int cbase = part * kChan;
      auto store_acc = [&](uint32_t col, const View &v) {
        static_assert(kBoxes == 1 || kChan % 32 == 0, "per-lane stores move 32 channels at a time");
        T *dst = static_cast<T *>(v.ptr) + v.offset(b, h, live ? xr : 0) + cbase;
#pragma unroll
        for (int c = 0; c < kChan; c += 32) {
          uint32_t r[32], pk[16];
          tmem_ld32(tlane + col + cbase + c, r);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) pk[i] = pack2<T>(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
          if (live) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              reinterpret_cast<uint4 *>(dst + c)[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
          }
        }
      };
      // D = 64: accumulators -> registers -> swizzled shared tiles -> one TMA store per tensor (coalesced, and rows
      // past the end are clipped by the hardware); per-lane 16-byte global stores are far slower.  The item's own
      // X tiles are dead by now (every MMA of the item has retired), so they serve as the staging tiles; the buffer
      // goes back to the producer only after the stores have read it (see `pending_xb`).  The barrier is executed
      // by every compute thread, whether or not its waits succeeded.
      const int xb = n % kXBuf;
      auto stage_acc = [&](uint32_t col, int which) {
        static_assert(kBoxes != 1 || kChan == 16 || kChan == 32, "staging moves 16 or 32 channels per thread");
        uint32_t r[kChan];
        if constexpr (kChan == 32) {
          tmem_ld32(tlane + col + cbase, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        } else {
          tmem_ld16(tlane + col + cbase, *reinterpret_cast<uint32_t(*)[16]>(&r[0]));
        }
        tc_wait_ld();
        unsigned char *tile = reinterpret_cast<unsigned char *>(s.x[xb][which][0]);
#pragma unroll
        for (int i = 0; i < kChan / 8; ++i) {
          uint4 v;
          v.x = pack2<T>(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
          v.y = pack2<T>(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
          v.z = pack2<T>(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
          v.w = pack2<T>(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
          *reinterpret_cast<uint4 *>(tile + swizzle128_offset(row, part * (kChan / 8) + i)) = v;
        }
      };
      if (kEarlyV) {
        if (ok && !__all_sync(0xffffffffu, mbar_wait_for(a.wait_cycles, &s.vdone, n & 1))) {
          atomicCAS(a.status, 0u, 214u);
          ok = false;
        }
        tc_fence_after();
        if (ok) {
          stage_acc(kColV, 2);
          if (has_t) stage_acc(kColVd, 3);
        }
      }
      if (ok && !__all_sync(0xffffffffu, mbar_wait_for(a.wait_cycles, &s.done, n & 1))) {
        atomicCAS(a.status, 0u, 206u);
        ok = false;
      }
      tc_fence_after();
      if (kBoxes == 1) {
        const bool w0 = kDoK, w1 = kDoK && has_t, w2 = kDoV, w3 = kDoV && has_t;
        if (ok) {
          if (w0) stage_acc(kColK, 0);
          if (w1) stage_acc(kColKd, 1);
          if (w2 && !kEarlyV) stage_acc(kColV, 2);
          if (w3 && !kEarlyV) stage_acc(kColVd, 3);
          fence_proxy_async();
        }
        asm volatile("bar.sync 2, %0;" ::"n"(kComputeThreads) : "memory");
        if (ctid == 0) {
          if (ok) {
            if (w0) tma_store_4d(&maps.out[0], s.x[xb][0][0], 0, x0, h, b);
            if (w1) tma_store_4d(&maps.out[1], s.x[xb][1][0], 0, x0, h, b);
            if (w2) tma_store_4d(&maps.out[2], s.x[xb][2][0], 0, x0, h, b);
            if (w3) tma_store_4d(&maps.out[3], s.x[xb][3][0], 0, x0, h, b);
            tma_store_commit();
          }
          pending_xb = xb;
        }
      } else if (ok) {
        if (kDoK) {
          store_acc(kColK, a.out[0]);
          if (has_t) store_acc(kColKd, a.out[1]);
        }
        if (kDoV) {
          store_acc(kColV, a.out[2]);
          if (has_t) store_acc(kColVd, a.out[3]);
        }
      }
      tc_fence_before();
      mbar_arrive(&s.acc_free);  // the next item may overwrite the accumulators
    }
   }  // items
  }

  if (threadIdx.x == 64) tma_store_wait_all();  // the thread that issued the output stores (nobody waits on x_empty any more)
  // A key-owner grid may finish before the query-owner grid it was allowed to start beside.  Work that follows the
  // call in the stream is ordered after this (the last) grid only, so one thread of every key-owner CTA waits for the
  // grid before it here: the call's completion then implies the query owner's (and, at head_dim 128, the first key
  // pass's).  Every CTA of the earlier grid is resident or done by the time a CTA of this one exists, so the wait
  // cannot deadlock; it costs nothing unless this grid really is the faster one.
  if (kKV && threadIdx.x == 32) griddep_wait();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

template <int D, int TILE, bool kKV, bool kDoK, bool kDoV, typename T>
cudaError_t launch_side(const BwdArgs &a, const float *delta, const float *dsum, cudaStream_t stream) {
  const bool has_t = a.g_to.ptr != nullptr, has_o = a.g_o.ptr != nullptr;
  const View qside[4] = {a.q, a.tq, a.g_to, a.g_o};
  const View kside[4] = {a.k, a.tk, a.v, a.tv};
  const View *xs = kKV ? kside : qside, *ys = kKV ? qside : kside;
  const int Lx = kKV ? a.Lk : a.Lq, Ly = kKV ? a.Lq : a.Lk;
  // which tensors each mode reads: the tangent-side ones only with a cotangent on Od, gO only when given
  const int qmask = 1 | (has_t ? 2 | 4 : 0) | (has_o ? 8 : 0);
  int kmask = 1 | (has_t ? 2 | 8 : 0) | 4;
  if (kKV && !kDoK) kmask &= 1 | 2;  // the dV / dVd pass of a split launch needs no value tiles
  BwdMaps maps;
  BwdKernelArgs ka{};
  ka.xmask = kKV ? kmask : qmask;
  ka.ymask = kKV ? qmask : kmask;
  for (int t = 0; t < 4; ++t) {
    if ((ka.xmask >> t & 1) &&
        !make_tensor_map(&maps.x[t], xs[t].ptr, a.dtype, a.B, a.H, Lx, D, xs[t].sb, xs[t].sh, xs[t].sl, kRows))
      return cudaErrorInvalidValue;
    if ((ka.ymask >> t & 1) &&
        !make_tensor_map(&maps.y[t], ys[t].ptr, a.dtype, a.B, a.H, Ly, D, ys[t].sb, ys[t].sh, ys[t].sl, TILE))
      return cudaErrorInvalidValue;
  }
  if (kKV) {
    ka.out[0] = a.dk; ka.out[1] = a.dtk; ka.out[2] = a.dv; ka.out[3] = a.dtv;
  } else {
    ka.out[0] = a.dq; ka.out[1] = a.dtq;
  }
  if (D == 64) {
    for (int t = 0; t < 4; ++t)
      if (ka.out[t].ptr &&
          !make_tensor_map(&maps.out[t], ka.out[t].ptr, a.dtype, a.B, a.H, Lx, D, ka.out[t].sb, ka.out[t].sh, ka.out[t].sl, kRows))
        return cudaErrorInvalidValue;
  }
  ka.lse = a.lse; ka.mu = a.mu; ka.delta = delta; ka.dsum = dsum; ka.status = a.status; ka.wait_cycles = a.wait_cycles;
  ka.B = a.B; ka.H = a.H; ka.Lx = Lx; ka.Ly = Ly; ka.Lq = a.Lq; ka.stat_len = a.stat_len;
  ka.has_t = has_t; ka.has_o = has_o; ka.scale = a.scale;
  auto kernel = sm100_bwd_kernel<D, TILE, kKV, kDoK, kDoV, T>;
  const size_t smem = sizeof(BwdSmem<D, TILE>) + 1024;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int64_t items = (int64_t)a.B * a.H * ((Lx + kRows - 1) / kRows);
  dim3 grid((unsigned)std::min<int64_t>(items, sm_count()));  // persistent: one CTA per SM walks the items
  {
    LaunchScope scope(kKV ? kIdBwdKeyTc : kIdBwdQueryTc, stream);
    e = launch_overlapped(kernel, grid, dim3(bwd_threads(bwd_parts(TILE))), smem, stream, maps, ka);
  }
  return e != cudaSuccess ? e : cudaGetLastError();
}

template <int D, typename T>
cudaError_t launch_bwd(const BwdArgs &a, cudaStream_t stream) {
  float *delta = static_cast<float *>(a.workspace);
  float *dsum = delta + (size_t)a.B * a.H * a.stat_len;
  {
    constexpr int kTpr = D / 8;
    const int64_t threads = (int64_t)a.B * a.H * a.Lq * kTpr;
    {
      LaunchScope scope(kIdRowDots, stream);
      row_dots_kernel<D, T><<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(a, delta, dsum);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  cudaError_t e = cudaSuccess;
  if constexpr (D == 64) {
    e = launch_side<D, 64, false, true, false, T>(a, delta, dsum, stream);
    if (e != cudaSuccess) return e;
    return launch_side<D, 64, true, true, true, T>(a, delta, dsum, stream);
  } else {
  // head_dim 128: four fp32 accumulators of 128 columns do not fit TMEM next to the score tiles, so the
  // key side runs as two passes (dK, dKd | dV, dVd) over 32-row query tiles
  e = launch_side<D, 32, false, true, false, T>(a, delta, dsum, stream);
  if (e != cudaSuccess) return e;
  e = launch_side<D, 32, true, true, false, T>(a, delta, dsum, stream);
  if (e != cudaSuccess) return e;
  return launch_side<D, 32, true, false, true, T>(a, delta, dsum, stream);
  }
}

}  // namespace

size_t sm100_bwd_workspace_bytes(int B, int H, int Lq, int Lk, int D, int stat_len) {
  (void)Lq; (void)Lk; (void)D;
  size_t bytes = (size_t)2 * B * H * stat_len * sizeof(float);
  return (bytes + 255) / 256 * 256;
}

bool sm100_bwd_supported(const BwdArgs &a) {
  if (a.D != 64 && a.D != 128) return false;
  if (a.Lq < 1 || a.Lk < 1 || a.H > 65535 || a.B > 65535) return false;
  const bool has_t = a.g_to.ptr != nullptr, has_o = a.g_o.ptr != nullptr;
  auto ok_q = [&](const View &v) { return tma_view_ok(v, a.B, a.H, a.Lq, a.D); };
  auto ok_k = [&](const View &v) { return tma_view_ok(v, a.B, a.H, a.Lk, a.D); };
  if (!ok_q(a.q) || !ok_q(a.o) || !ok_q(a.dq) || !ok_k(a.k) || !ok_k(a.v) || !ok_k(a.dk) || !ok_k(a.dv)) return false;
  if (has_t && (!ok_q(a.tq) || !ok_q(a.to) || !ok_q(a.g_to) || !ok_q(a.dtq) || !ok_k(a.tk) || !ok_k(a.tv) || !ok_k(a.dtk) ||
                !ok_k(a.dtv)))
    return false;
  if (has_o && !ok_q(a.g_o)) return false;
  // the query owner's row statistics travel by 16-byte-granular bulk copies
  if (reinterpret_cast<uintptr_t>(a.lse) % 16 || reinterpret_cast<uintptr_t>(a.workspace) % 16 || a.stat_len % 4) return false;
  if (has_t && reinterpret_cast<uintptr_t>(a.mu) % 16) return false;
  return true;
}

cudaError_t sm100_bwd(const BwdArgs &a, cudaStream_t stream) {
  if (a.dtype == JVPATTN_BF16)
    return a.D == 64 ? launch_bwd<64, __nv_bfloat16>(a, stream) : launch_bwd<128, __nv_bfloat16>(a, stream);
  return a.D == 64 ? launch_bwd<64, __half>(a, stream) : launch_bwd<128, __half>(a, stream);
}

}  // namespace jvpattn
