// Shared declarations of the jvpattn kernels: the validated problem description that the C-ABI layer
// hands to the kernel launchers, and small device helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/jvpattn.h"

namespace jvpattn {

// A (B,H,L,D) view with unit innermost stride.  Strides are in elements.
struct View {
  void *ptr;
  int64_t sb, sh, sl;
  __host__ __device__ __forceinline__ int64_t offset(int b, int h, int l) const {
    return (int64_t)b * sb + (int64_t)h * sh + (int64_t)l * sl;
  }
};

struct FwdArgs {
  View q, k, v, tq, tk, tv, o, to;
  float *lse, *mu, *li;  // li may be null
  unsigned int *status;  // device status word, set when a bounded wait runs out
  long long wait_cycles; // budget of every device-side wait, in clock cycles
  int inject;            // test hook: 1 = the producer over-declares the bytes of the first key tile (its barrier never completes)
  int has_t;             // 0: primal only (tq, tk, tv alias q, k, v; to.ptr and mu are null and not written)
  int B, H, Lq, Lk, D, stat_len;
  int dtype;
  float scale;
};

struct BwdArgs {
  View q, k, v, tq, tk, tv, o, to;
  View g_o, g_to;  // ptr == nullptr when the cotangent is absent
  View dq, dk, dv, dtq, dtk, dtv;
  const float *lse, *mu;
  void *workspace;
  size_t workspace_bytes;
  unsigned int *status;
  long long wait_cycles;
  int B, H, Lq, Lk, D, stat_len;
  int dtype;
  float scale;
};

// launchers (each returns a cudaError_t from the launch; they never synchronise)
cudaError_t simt_fwd(const FwdArgs &a, cudaStream_t stream);
cudaError_t simt_bwd(const BwdArgs &a, cudaStream_t stream);

bool sm100_fwd_supported(const FwdArgs &a);
bool sm100_bwd_supported(const BwdArgs &a);
cudaError_t sm100_fwd(const FwdArgs &a, cudaStream_t stream);
cudaError_t sm100_bwd(const BwdArgs &a, cudaStream_t stream);
size_t sm100_bwd_workspace_bytes(int B, int H, int Lq, int Lk, int D, int stat_len);
// rotary.cu: rotation by fixed angles fused with the cast (dtype codes 0 bf16, 1 fp16, 2 fp32)
cudaError_t rotary_cast(const void *x, int64_t sb, int64_t ss, int64_t sh, int in_dtype, void *y, int out_dtype,
                        const float *cosv, const float *sinv, int B, int S, int H, int D, int transpose, cudaStream_t stream);

cudaError_t rotary_qkv(const void *const in[3], const int64_t in_strides[9], int in_dtype, void *const out[3],
                       const int64_t out_strides[9], int out_dtype, const float *cosv, const float *sinv, int B, int S, int H, int D,
                       int transpose, cudaStream_t stream);

// dual_pointwise.cu: LayerNorm + modulation and gated residual on (primal, tangent) pairs, with their VJPs
bool dual_shape_ok(int B, int S, int C);
cudaError_t ln_modulate(int which, const void *x, const void *tx, const float *gamma, const float *beta, const void *shift,
                        const void *scale, const void *tshift, const void *tscale, int64_t mod_stride, int64_t tmod_stride,
                        float *mean, float *rstd, void *out, const void *g, void *dx, void *dtx, float *sums, int B, int S, int C,
                        float eps, int exact, int dtype, cudaStream_t stream);
cudaError_t gated_residual(const void *x, const void *y, const void *gate, const void *mask, int64_t gate_stride, void *z, int B,
                           int S, int C, int dtype, const unsigned long long *drop_seed, unsigned drop_call, float drop_p,
                           cudaStream_t stream);
cudaError_t ln_finalize(const float *p, const float *t, const float *gamma, const float *beta, const void *scale,
                        const void *tscale, int64_t mod_stride, int64_t tmod_stride, void *d_shift, void *d_scale, void *d_tshift,
                        void *d_tscale, float *d_gamma, float *d_beta, int B, int C, int dtype, cudaStream_t stream);
cudaError_t gated_residual_dual(int which, const void *x, const void *tx, const void *y, const void *ty, const void *gate,
                                const void *tgate, const void *mask, int64_t gate_stride, int64_t tgate_stride, void *z, void *tz,
                                const void *gz, const void *gtz, void *d_y, void *d_ty, float *sums, int B, int S, int C, int dtype,
                                const unsigned long long *drop_seed, unsigned drop_call, float drop_p, cudaStream_t stream);
cudaError_t gelu_dual(int mode, const void *h, const void *v, const void *w, const void *u, void *out, void *out2, int64_t n,
                      int dtype, cudaStream_t stream);

// vocab_loss.cu: interpolation, flow map, cross-entropy and self-distillation loss over the vocabulary axis
cudaError_t vocab_loss(int op, const void *l, const void *tl, const void *lt, int64_t ld, const float *x0, int64_t ldx,
                       const int64_t *ids, const float *s, const float *t, float *lse, float *stats, float *loss, const float *g,
                       void *out, void *out2, int64_t ldo, float eps, int batch, int rows_per_sample, int V, int dtype,
                       cudaStream_t stream);

// vocab_head.cu: flow-map head over the vocabulary axis on (primal, tangent) pairs, with its VJPs
cudaError_t vocab_head(int which, const void *l, const void *tl, int64_t ldl, int64_t ldt, const float *x, const float *dt,
                       const float *ddt, float *lse, float *out, const float *g, void *dl, void *dtl, int batch,
                       int rows_per_sample, int V, int dtype, cudaStream_t stream);

// Kernel identifiers used by the launch counter and the optional per-kernel event timing.
enum KernelId {
  kIdFwdTc = 0, kIdRowDots, kIdBwdQueryTc, kIdBwdKeyTc, kIdFwdSimt, kIdBwdQuerySimt, kIdBwdKeySimt, kIdRotary, kIdDual, kNumKernelIds
};

// Brackets one kernel launch: counts it and, while profiling is on, records a CUDA event before and
// after it on the launching stream.
struct LaunchScope {
  LaunchScope(int id, cudaStream_t stream);
  ~LaunchScope();
  int id_;
  cudaStream_t stream_;
  void *slot_;
};

// Launch with the programmatic-serialization attribute: the kernel may start as soon as the kernel before it in
// the stream has released its dependents (see griddep_launch_dependents), without waiting for it to finish.
template <typename... Params, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

template <typename T> struct Elem;
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
};

}  // namespace jvpattn
