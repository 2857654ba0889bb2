// extern "C" entry points of libjvpattn: argument validation, kernel-family selection, launch.
// No torch types, no device allocation, no host synchronisation (except jvpattn_device_status).
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "jvpattn_common.cuh"
#include "sm100_ptx.cuh"

namespace jvpattn {

static std::atomic<uint64_t> g_launches{0};
// Test hooks (jvpattn_debug_set): the budget of the device-side waits and a one-shot injection for the next forward.
static std::atomic<long long> g_wait_cycles{ptx::kWaitCycles};
static std::atomic<int> g_inject_fwd{0};

// ---- optional per-kernel timing (off by default; used by bench.py for the roofline figures)
struct ProfSlot {
  int id;
  cudaEvent_t start, stop;
};
static std::atomic<bool> g_profiling{false};
static std::mutex g_prof_mutex;
static std::vector<ProfSlot *> g_prof_slots;

LaunchScope::LaunchScope(int id, cudaStream_t stream) : id_(id), stream_(stream), slot_(nullptr) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (!g_profiling.load(std::memory_order_relaxed)) return;
  ProfSlot *slot = new ProfSlot{id, nullptr, nullptr};
  if (cudaEventCreate(&slot->start) != cudaSuccess || cudaEventCreate(&slot->stop) != cudaSuccess) {
    (void)cudaGetLastError();
    delete slot;
    return;
  }
  cudaEventRecord(slot->start, stream);
  slot_ = slot;
}

LaunchScope::~LaunchScope() {
  if (!slot_) return;
  ProfSlot *slot = static_cast<ProfSlot *>(slot_);
  cudaEventRecord(slot->stop, stream_);
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  g_prof_slots.push_back(slot);
}

// Written by a kernel whose bounded wait ran out; read and cleared by jvpattn_device_status().
__device__ unsigned int g_status_word = 0;

namespace {

thread_local char t_cuda_error[256] = "";

constexpr int kMaxDevices = 64;
struct DeviceInfo {
  int state = 0;  // 0 unknown, 1 usable sm_100, -1 unusable
  unsigned int *status = nullptr;
};
DeviceInfo g_devices[kMaxDevices];
std::mutex g_device_mutex;

int note_cuda(cudaError_t e) {
  if (e == cudaSuccess) return JVPATTN_OK;
  std::snprintf(t_cuda_error, sizeof(t_cuda_error), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
  (void)cudaGetLastError();
  return JVPATTN_ELAUNCH;
}

// Resolves the current device once: compute capability and the address of its status word.
int current_device(DeviceInfo **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    note_cuda(e);
    return JVPATTN_EARCH;
  }
  std::lock_guard<std::mutex> lock(g_device_mutex);
  DeviceInfo &d = g_devices[dev];
  if (d.state == 0) {
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess || major != 10) {
      note_cuda(e);
      d.state = -1;
    } else {
      void *p = nullptr;
      e = cudaGetSymbolAddress(&p, g_status_word);
      if (e != cudaSuccess) {
        note_cuda(e);
        d.state = -1;
      } else {
        d.status = static_cast<unsigned int *>(p);
        d.state = 1;
      }
    }
  }
  if (d.state != 1) return JVPATTN_EARCH;
  *out = &d;
  return JVPATTN_OK;
}

int check_problem(const jvpattn_problem *p) {
  if (!p) return JVPATTN_EINVAL;
  if (p->batch < 0 || p->heads < 0 || p->len_q < 0 || p->len_k < 0) return JVPATTN_EINVAL;
  if (p->dtype != JVPATTN_BF16 && p->dtype != JVPATTN_FP16) return JVPATTN_EINVAL;
  if (p->kernels < JVPATTN_KERNELS_AUTO || p->kernels > JVPATTN_KERNELS_TCGEN05) return JVPATTN_EINVAL;
  if (p->head_dim < 16 || p->head_dim > 128) return JVPATTN_EHEADDIM;
  if (p->stat_len < p->len_q || p->stat_len % 128 != 0) return JVPATTN_ESTAT;
  if (p->len_k == 0 && p->len_q > 0 && p->batch > 0 && p->heads > 0) return JVPATTN_EINVAL;  // softmax over nothing
  if (!(p->scale == p->scale)) return JVPATTN_EINVAL;
  return JVPATTN_OK;
}

bool is_empty(const jvpattn_problem *p) { return p->batch == 0 || p->heads == 0 || (p->len_q == 0 && p->len_k == 0); }

int to_view(const jvpattn_tensor *t, bool required, View *v) {
  if (!t || !t->ptr) {
    if (required) return JVPATTN_EINVAL;
    *v = View{nullptr, 0, 0, 0};
    return JVPATTN_OK;
  }
  if (t->stride[3] != 1) return JVPATTN_ESTRIDE;
  if (reinterpret_cast<uintptr_t>(t->ptr) % 2 != 0) return JVPATTN_EALIGN;
  *v = View{t->ptr, t->stride[0], t->stride[1], t->stride[2]};
  return JVPATTN_OK;
}

float effective_scale(const jvpattn_problem *p) {
  return p->scale > 0.f ? p->scale : 1.0f / std::sqrt((float)p->head_dim);
}

#define JVP_TRY(expr)            \
  do {                           \
    int rc__ = (expr);           \
    if (rc__ != JVPATTN_OK) return rc__; \
  } while (0)

int build_fwd(const jvpattn_problem *p, const jvpattn_tensor *q, const jvpattn_tensor *k, const jvpattn_tensor *v,
              const jvpattn_tensor *tq, const jvpattn_tensor *tk, const jvpattn_tensor *tv,
              const jvpattn_tensor *o, const jvpattn_tensor *to, float *lse, float *mu, float *li, FwdArgs *a) {
  JVP_TRY(check_problem(p));
  JVP_TRY(to_view(q, true, &a->q));
  JVP_TRY(to_view(k, true, &a->k));
  JVP_TRY(to_view(v, true, &a->v));
  // tangents: all four of tq, tk, tv, to (and mu), or none of them (primal-only attention)
  const bool any_t = (tq && tq->ptr) || (tk && tk->ptr) || (tv && tv->ptr) || (to && to->ptr);
  JVP_TRY(to_view(tq, any_t, &a->tq));
  JVP_TRY(to_view(tk, any_t, &a->tk));
  JVP_TRY(to_view(tv, any_t, &a->tv));
  JVP_TRY(to_view(o, true, &a->o));
  JVP_TRY(to_view(to, any_t, &a->to));
  if (!lse || (any_t && !mu)) return JVPATTN_EINVAL;
  if (!any_t) {
    // kernels that walk all six inputs (the portable ones) read the primals twice; nothing of it is written
    a->tq = a->q; a->tk = a->k; a->tv = a->v;
    mu = nullptr;
  }
  a->has_t = any_t ? 1 : 0;
  a->lse = lse; a->mu = mu; a->li = li;
  a->B = p->batch; a->H = p->heads; a->Lq = p->len_q; a->Lk = p->len_k; a->D = p->head_dim;
  a->stat_len = p->stat_len; a->dtype = p->dtype; a->scale = effective_scale(p);
  a->status = nullptr;
  a->wait_cycles = g_wait_cycles.load(std::memory_order_relaxed);
  a->inject = 0;
  return JVPATTN_OK;
}

int build_bwd(const jvpattn_problem *p, const jvpattn_tensor *q, const jvpattn_tensor *k, const jvpattn_tensor *v,
              const jvpattn_tensor *tq, const jvpattn_tensor *tk, const jvpattn_tensor *tv,
              const jvpattn_tensor *o, const jvpattn_tensor *to, const jvpattn_tensor *g_o, const jvpattn_tensor *g_to,
              const float *lse, const float *mu, const jvpattn_tensor *dq, const jvpattn_tensor *dk,
              const jvpattn_tensor *dv, const jvpattn_tensor *dtq, const jvpattn_tensor *dtk, const jvpattn_tensor *dtv,
              BwdArgs *a) {
  JVP_TRY(check_problem(p));
  JVP_TRY(to_view(g_o, false, &a->g_o));
  JVP_TRY(to_view(g_to, false, &a->g_to));
  if (!a->g_o.ptr && !a->g_to.ptr) return JVPATTN_EINVAL;
  const bool need_t = a->g_to.ptr != nullptr;
  JVP_TRY(to_view(q, true, &a->q));
  JVP_TRY(to_view(k, true, &a->k));
  JVP_TRY(to_view(v, true, &a->v));
  JVP_TRY(to_view(o, true, &a->o));
  JVP_TRY(to_view(tq, need_t, &a->tq));
  JVP_TRY(to_view(tk, need_t, &a->tk));
  JVP_TRY(to_view(tv, need_t, &a->tv));
  JVP_TRY(to_view(to, need_t, &a->to));
  JVP_TRY(to_view(dq, true, &a->dq));
  JVP_TRY(to_view(dk, true, &a->dk));
  JVP_TRY(to_view(dv, true, &a->dv));
  JVP_TRY(to_view(dtq, need_t, &a->dtq));
  JVP_TRY(to_view(dtk, need_t, &a->dtk));
  JVP_TRY(to_view(dtv, need_t, &a->dtv));
  if (!lse || (need_t && !mu)) return JVPATTN_EINVAL;
  if (!need_t) {
    // Without a cotangent on the tangent output nothing depends on the tangents or on mu: every term
    // they enter is multiplied by an exact zero.  Point the unused views at valid memory.
    a->tq = a->q; a->tk = a->k; a->tv = a->v; a->to = a->o;
    a->dtq = a->dtk = a->dtv = View{nullptr, 0, 0, 0};
    mu = lse;
  }
  a->lse = lse; a->mu = mu;
  a->B = p->batch; a->H = p->heads; a->Lq = p->len_q; a->Lk = p->len_k; a->D = p->head_dim;
  a->stat_len = p->stat_len; a->dtype = p->dtype; a->scale = effective_scale(p);
  a->workspace = nullptr; a->workspace_bytes = 0; a->status = nullptr;
  a->wait_cycles = g_wait_cycles.load(std::memory_order_relaxed);
  return JVPATTN_OK;
}

}  // namespace
}  // namespace jvpattn

using namespace jvpattn;

extern "C" {

int jvpattn_abi_version(void) { return JVPATTN_ABI_VERSION; }

int jvpattn_rotary_cast(const void *x, int64_t sb, int64_t ss, int64_t sh, int in_dtype, void *y, int out_dtype,
                        const float *cosv, const float *sinv, int batch, int len, int heads, int head_dim, int transpose,
                        void *stream) {
  if (batch < 0 || len < 0 || heads < 0 || head_dim < 16 || head_dim % 16 != 0) return JVPATTN_EINVAL;
  if (in_dtype < 0 || in_dtype > JVPATTN_FP32 || out_dtype < 0 || out_dtype > JVPATTN_FP32) return JVPATTN_EINVAL;
  DeviceInfo *d = nullptr;
  if (int rc = current_device(&d)) return rc;
  if ((int64_t)batch * len * heads == 0) return JVPATTN_OK;
  if (!x || !y || !cosv || !sinv) return JVPATTN_EINVAL;
  return note_cuda(rotary_cast(x, sb, ss, sh, in_dtype, y, out_dtype, cosv, sinv, batch, len, heads, head_dim, transpose,
                               static_cast<cudaStream_t>(stream)));
}

int jvpattn_rotary_qkv(const void *const in[3], const int64_t in_strides[9], int in_dtype, void *const out[3],
                       const int64_t out_strides[9], int out_dtype, const float *cosv, const float *sinv, int batch, int len,
                       int heads, int head_dim, int transpose, void *stream) {
  if (batch < 0 || len < 0 || heads < 0 || head_dim < 16 || head_dim % 16 != 0) return JVPATTN_EINVAL;
  if ((in_dtype != JVPATTN_BF16 && in_dtype != JVPATTN_FP32) || (out_dtype != JVPATTN_BF16 && out_dtype != JVPATTN_FP32))
    return JVPATTN_EINVAL;
  DeviceInfo *d = nullptr;
  if (int rc = current_device(&d)) return rc;
  if ((int64_t)batch * len * heads == 0) return JVPATTN_OK;
  if (!in || !out || !in_strides || !out_strides || !cosv || !sinv) return JVPATTN_EINVAL;
  if (reinterpret_cast<uintptr_t>(cosv) % 16 || reinterpret_cast<uintptr_t>(sinv) % 16) return JVPATTN_EALIGN;
  for (int t = 0; t < 3; ++t) {
    if (!in[t] || !out[t]) return JVPATTN_EINVAL;
    if (reinterpret_cast<uintptr_t>(in[t]) % 16 || reinterpret_cast<uintptr_t>(out[t]) % 16) return JVPATTN_EALIGN;
    for (int k = 0; k < 3; ++k)
      if (in_strides[3 * t + k] % 8 || out_strides[3 * t + k] % 8) return JVPATTN_EALIGN;
  }
  return note_cuda(rotary_qkv(in, in_strides, in_dtype, out, out_strides, out_dtype, cosv, sinv, batch, len, heads, head_dim,
                              transpose, static_cast<cudaStream_t>(stream)));
}

int jvpattn_ln_modulate(int which, const void *x, const void *tx, const float *gamma, const float *beta, const void *shift,
                        const void *scale, const void *tshift, const void *tscale, int64_t mod_stride, int64_t tmod_stride,
                        float *mean, float *rstd, void *out, const void *g, void *dx, void *dtx, float *sums, int batch, int len,
                        int channels, float eps, int exact, int dtype, void *stream) {
  if (which < 0 || which > 3 || !dual_shape_ok(batch, len, channels)) return JVPATTN_EINVAL;
  if (dtype != JVPATTN_BF16 && dtype != JVPATTN_FP32) return JVPATTN_EINVAL;
  DeviceInfo *d = nullptr;
  if (int rc = current_device(&d)) return rc;
  if ((int64_t)batch * len == 0) return JVPATTN_OK;
  if (!x || !gamma || !scale || !mean || !rstd) return JVPATTN_EINVAL;
  if ((which == 0 && (!shift || !out)) || (which == 1 && (!tx || !out)) || (which >= 2 && (!g || !dx || !sums)) ||
      (which == 3 && (!tx || !dtx)))
    return JVPATTN_EINVAL;
  if (mod_stride % 8 || tmod_stride % 8) return JVPATTN_EALIGN;
  return note_cuda(ln_modulate(which, x, tx, gamma, beta, shift, scale, tshift, tscale, mod_stride, tmod_stride, mean, rstd, out, g,
                               dx, dtx, sums, batch, len, channels, eps, exact, dtype, static_cast<cudaStream_t>(stream)));
}

int jvpattn_gated_residual(const void *x, const void *y, const void *gate, const void *mask, int64_t gate_stride, void *z,
                           int batch, int len, int channels, int dtype, const jvpattn_dropout *drop, void *stream) {
  if (batch < 0 || len < 0 || channels < 8 || channels % 8) return JVPATTN_EINVAL;
  if (dtype != JVPATTN_BF16 && dtype != JVPATTN_FP32) return JVPATTN_EINVAL;
  if (drop && (!drop->seed || !(drop->p >= 0.f) || !(drop->p < 1.f))) return JVPATTN_EINVAL;
  DeviceInfo *d = nullptr;
  if (int rc = current_device(&d)) return rc;
  if ((int64_t)batch * len == 0) return JVPATTN_OK;
  if (!x || !y || !gate || !z) return JVPATTN_EINVAL;
  for (const void *p : {x, y, gate, mask, (const void *)z})
    if (p && reinterpret_cast<uintptr_t>(p) % 16) return JVPATTN_EALIGN;
  if (gate_stride % 8) return JVPATTN_EALIGN;
  return note_cuda(gated_residual(x, y, gate, mask, gate_stride, z, batch, len, channels, dtype,
                                  drop ? reinterpret_cast<const unsigned long long *>(drop->seed) : nullptr,
                                  drop ? drop->call : 0u, drop ? drop->p : 0.f, static_cast<cudaStream_t>(stream)));
}

int jvpattn_flow_map_head(int which, const void *logits, const void *tlogits, int64_t ld_logits, int64_t ld_tlogits, const float *x,
                          const float *dt, const float *ddt, float *lse, float *out, const float *g, void *dlogits,
                          void *dtlogits, int batch, int rows_per_sample, int vocab, int dtype, void *stream) {
  if (which < 0 || which > 3 || batch < 0 || rows_per_sample < 0 || vocab < 1) return JVPATTN_EINVAL;
  if (dtype != JVPATTN_BF16 && dtype != JVPATTN_FP32) return JVPATTN_EINVAL;
  if ((size_t)((vocab + 7) & ~7) * (dtype == JVPATTN_BF16 ? 4 : 8) > 200 * 1024) return JVPATTN_EINVAL;  // the row pair must fit shared memory
  DeviceInfo *d = nullptr;
  if (int rc = current_device(&d)) return rc;
  if ((int64_t)batch * rows_per_sample == 0) return JVPATTN_OK;
  if (!logits || !dt || !lse) return JVPATTN_EINVAL;
  if ((which == 0 && (!x || !out)) || (which == 1 && (!x || !out || !tlogits || !ddt)) || (which == 2 && (!g || !dlogits)) ||
      (which == 3 && (!g || !dlogits || !dtlogits || !tlogits || !ddt)))
    return JVPATTN_EINVAL;
  return note_cuda(vocab_head(which, logits, tlogits, ld_logits, ld_tlogits, x, dt, ddt, lse, out, g, dlogits, dtlogits, batch,
                              rows_per_sample, vocab, dtype, static_cast<cudaStream_t>(stream)));
}

int jvpattn_gelu_dual(int mode, const void *h, const void *v, const void *w, const void *u, void *out, void *out2, int64_t n,
                      int dtype, void *stream) {
  if (mode < 0 || mode > 4 || n < 0 || n % 8) return JVPATTN_EINVAL;
  if (dtype != JVPATTN_BF16 && dtype != JVPATTN_FP32) return JVPATTN_EINVAL;
  DeviceInfo *d = nullptr;
  if (int rc = current_device(&d)) return rc;
  if (n == 0) return JVPATTN_OK;
  if (!h || !out || (mode >= 1 && !v) || (mode >= 2 && !out2) || ((mode == 2 || mode == 4) && !w) || (mode == 4 && !u))
    return JVPATTN_EINVAL;
  for (const void *p : {h, v, w, u, (const void *)out, (const void *)out2})
    if (p && reinterpret_cast<uintptr_t>(p) % 16) return JVPATTN_EALIGN;
  return note_cuda(gelu_dual(mode, h, v, w, u, out, out2, n, dtype, static_cast<cudaStream_t>(stream)));
}

int jvpattn_ln_finalize(const float *sums_y, const float *sums_ty, const float *gamma, const float *beta, const void *scale,
                        const void *tscale, int64_t mod_stride, int64_t tmod_stride, void *d_shift, void *d_scale, void *d_tshift,
                        void *d_tscale, float *d_gamma, float *d_beta, int batch, int channels, int dtype, void *stream) {
  if (batch < 0 || channels < 0) return JVPATTN_EINVAL;
  if (dtype != JVPATTN_BF16 && dtype != JVPATTN_FP32) return JVPATTN_EINVAL;
  DeviceInfo *d = nullptr;
  if (int rc = current_device(&d)) return rc;
  if (!gamma || !scale || !d_gamma || (!sums_y && !sums_ty)) return JVPATTN_EINVAL;
  return note_cuda(ln_finalize(sums_y, sums_ty, gamma, beta, scale, tscale, mod_stride, tmod_stride, d_shift, d_scale, d_tshift,
                               d_tscale, d_gamma, d_beta, batch, channels, dtype, static_cast<cudaStream_t>(stream)));
}

int jvpattn_gated_residual_dual(int which, const void *x, const void *tx, const void *y, const void *ty, const void *gate,
                                const void *tgate, const void *mask, int64_t gate_stride, int64_t tgate_stride, void *z, void *tz,
                                const void *gz, const void *gtz, void *d_y, void *d_ty, float *sums, int batch, int len,
                                int channels, int dtype, const jvpattn_dropout *drop, void *stream) {
  if (drop && (!drop->seed || !(drop->p >= 0.f) || !(drop->p < 1.f))) return JVPATTN_EINVAL;
  if (which < 0 || which > 1 || batch < 0 || len < 0 || channels < 8 || channels % 8 || channels > 1024) return JVPATTN_EINVAL;
  if (dtype != JVPATTN_BF16 && dtype != JVPATTN_FP32) return JVPATTN_EINVAL;
  DeviceInfo *d = nullptr;
  if (int rc = current_device(&d)) return rc;
  if ((int64_t)batch * len == 0) return JVPATTN_OK;
  if (!y || !gate) return JVPATTN_EINVAL;
  if (which == 0 && (!x || !z || !tz)) return JVPATTN_EINVAL;
  if (which == 1 && ((!gz && !gtz) || !d_y || !sums || (gtz && !d_ty))) return JVPATTN_EINVAL;
  for (const void *p : {x, tx, y, ty, gate, tgate, mask, (const void *)z, (const void *)tz, gz, gtz, (const void *)d_y, (const void *)d_ty})
    if (p && reinterpret_cast<uintptr_t>(p) % 16) return JVPATTN_EALIGN;
  if (gate_stride % 8 || tgate_stride % 8) return JVPATTN_EALIGN;
  return note_cuda(gated_residual_dual(which, x, tx, y, ty, gate, tgate, mask, gate_stride, tgate_stride, z, tz, gz, gtz, d_y, d_ty,
                                       sums, batch, len, channels, dtype,
                                       drop ? reinterpret_cast<const unsigned long long *>(drop->seed) : nullptr,
                                       drop ? drop->call : 0u, drop ? drop->p : 0.f, static_cast<cudaStream_t>(stream)));
}

int jvpattn_vocab_op(int op, const void *logits, const void *tlogits, const void *target_logits, int64_t ld, const float *x0,
                     int64_t ldx, const int64_t *ids, const float *s, const float *t, float *lse, float *stats, float *loss,
                     const float *g, void *out, void *out2, int64_t ldo, float eps, int batch, int rows_per_sample, int vocab,
                     int dtype, void *stream) {
  if (op < 0 || op > 5 || batch < 0 || rows_per_sample < 0 || vocab < 1) return JVPATTN_EINVAL;
  if (dtype != JVPATTN_BF16 && dtype != JVPATTN_FP32) return JVPATTN_EINVAL;
  DeviceInfo *d = nullptr;
  if (int rc = current_device(&d)) return rc;
  if ((int64_t)batch * rows_per_sample == 0) return JVPATTN_OK;
  const bool ok = op == 0   ? x0 && ids && t && out
                  : op == 1 ? logits && x0 && ids && s && t && lse && out
                  : op == 2 ? logits && ids && lse && loss
                  : op == 3 ? logits && ids && lse && g && out
                  : op == 4 ? logits && tlogits && target_logits && x0 && ids && s && t && lse && stats && loss
                            : logits && tlogits && target_logits && x0 && ids && s && t && lse && stats && g && out && out2;
  if (!ok) return JVPATTN_EINVAL;
  return note_cuda(vocab_loss(op, logits, tlogits, target_logits, ld, x0, ldx, ids, s, t, lse, stats, loss, g, out, out2, ldo,
                              eps, batch, rows_per_sample, vocab, dtype, static_cast<cudaStream_t>(stream)));
}

uint64_t jvpattn_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char *jvpattn_last_cuda_error(void) { return t_cuda_error; }

const char *jvpattn_strerror(int code) {
  switch (code) {
    case JVPATTN_OK: return "ok";
    case JVPATTN_EINVAL: return "invalid argument (null tensor, negative size, empty key axis, unknown dtype or kernel family, or a shape the forced kernel family cannot run)";
    case JVPATTN_ESTRIDE: return "innermost stride must be 1";
    case JVPATTN_EALIGN: return "pointer or stride alignment not supported";
    case JVPATTN_EHEADDIM: return "head_dim must be in [16, 128]";
    case JVPATTN_ESTAT: return "row-statistic length must be a multiple of 128 and >= len_q";
    case JVPATTN_EWORKSPACE: return "workspace missing or too small (see jvpattn_bwd_workspace_bytes)";
    case JVPATTN_EARCH: return "no usable CUDA device: this library runs on sm_100 (B200) only and has no CPU path";
    case JVPATTN_ELAUNCH: return "CUDA launch failed (see jvpattn_last_cuda_error)";
    case JVPATTN_EDEVICE: return "a bounded device-side wait ran out (jvpattn_device_status gives the code of the wait)";
    case JVPATTN_ETOOLARGE: return "problem exceeds the built-in scratch of jvpattn_bwd_static (batch*heads*stat_len > JVPATTN_STATIC_SCRATCH_ROWS); use jvpattn_bwd with a caller workspace";
    default: return "unknown jvpattn error code";
  }
}

int jvpattn_profile_begin(void) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  g_profiling.store(true);
  return JVPATTN_OK;
}

int jvpattn_profile_end(double *total_ms, uint64_t *launches) {
  g_profiling.store(false);
  cudaError_t e = cudaDeviceSynchronize();
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  for (int i = 0; i < JVPATTN_NUM_KERNELS; ++i) {
    if (total_ms) total_ms[i] = 0.0;
    if (launches) launches[i] = 0;
  }
  for (ProfSlot *slot : g_prof_slots) {
    float ms = 0.f;
    if (e == cudaSuccess && cudaEventElapsedTime(&ms, slot->start, slot->stop) == cudaSuccess && slot->id >= 0 &&
        slot->id < JVPATTN_NUM_KERNELS) {
      if (total_ms) total_ms[slot->id] += ms;
      if (launches) launches[slot->id] += 1;
    }
    cudaEventDestroy(slot->start);
    cudaEventDestroy(slot->stop);
    delete slot;
  }
  g_prof_slots.clear();
  (void)cudaGetLastError();
  return e == cudaSuccess ? JVPATTN_OK : note_cuda(e);
}

const char *jvpattn_kernel_name(int id) {
  static_assert(kNumKernelIds == JVPATTN_NUM_KERNELS, "kernel id table");
  switch (id) {
    case kIdFwdTc: return "sm100_fwd_kernel";
    case kIdRowDots: return "row_dots_kernel";
    case kIdBwdQueryTc: return "sm100_bwd_kernel<query owner>";
    case kIdBwdKeyTc: return "sm100_bwd_kernel<key owner>";
    case kIdFwdSimt: return "simt_fwd_kernel";
    case kIdBwdQuerySimt: return "simt_bwd_q_kernel";
    case kIdBwdKeySimt: return "simt_bwd_kv_kernel";
    case kIdRotary: return "rotary_cast_kernel";
    case kIdDual: return "dual_pointwise_kernels";
    default: return "?";
  }
}

int jvpattn_device_status(void) {
  DeviceInfo *d = nullptr;
  int rc = current_device(&d);
  if (rc != JVPATTN_OK) return rc;
  unsigned int word = 0, zero = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(&word, d->status, sizeof(word), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && word != 0) e = cudaMemcpy(d->status, &zero, sizeof(zero), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return note_cuda(e);
  return (int)word;
}

int jvpattn_stream_check(void *stream) {
  DeviceInfo *d = nullptr;
  int rc = current_device(&d);
  if (rc != JVPATTN_OK) return rc;
  unsigned int word = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(&word, d->status, sizeof(word), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return note_cuda(e);
  return word != 0 ? JVPATTN_EDEVICE : JVPATTN_OK;
}

int jvpattn_debug_set(int knob, long long value) {
  switch (knob) {
    case JVPATTN_DEBUG_WAIT_CYCLES:
      g_wait_cycles.store(value > 0 ? value : ptx::kWaitCycles);
      return JVPATTN_OK;
    case JVPATTN_DEBUG_STALL_NEXT_FWD:
      g_inject_fwd.store(value != 0 ? 1 : 0);
      return JVPATTN_OK;
    default:
      return JVPATTN_EINVAL;
  }
}

int jvpattn_selected_kernels(const jvpattn_problem *p, int which) {
  int rc = check_problem(p);
  if (rc != JVPATTN_OK) return rc;
  if (p->kernels != JVPATTN_KERNELS_AUTO) return p->kernels;
  // Shape-only decision with ideally aligned tensors; a misaligned call still falls back to SIMT.
  if (which == 0) {
    FwdArgs a{};
    a.B = p->batch; a.H = p->heads; a.Lq = p->len_q; a.Lk = p->len_k; a.D = p->head_dim; a.dtype = p->dtype;
    a.stat_len = p->stat_len;
    const int64_t sl = p->head_dim;
    a.q = a.k = a.v = a.tq = a.tk = a.tv = a.o = a.to = View{(void *)16, sl * p->len_q, sl * p->len_q * p->batch, sl};
    return sm100_fwd_supported(a) ? JVPATTN_KERNELS_TCGEN05 : JVPATTN_KERNELS_SIMT;
  }
  BwdArgs a{};
  a.B = p->batch; a.H = p->heads; a.Lq = p->len_q; a.Lk = p->len_k; a.D = p->head_dim; a.dtype = p->dtype;
  a.stat_len = p->stat_len;
  const int64_t sl = p->head_dim;
  View any{(void *)16, sl * p->len_q, sl * p->len_q * p->batch, sl};
  a.q = a.k = a.v = a.tq = a.tk = a.tv = a.o = a.to = a.g_o = a.g_to = a.dq = a.dk = a.dv = a.dtq = a.dtk = a.dtv = any;
  return sm100_bwd_supported(a) ? JVPATTN_KERNELS_TCGEN05 : JVPATTN_KERNELS_SIMT;
}

int jvpattn_fwd(const jvpattn_problem *p, const jvpattn_tensor *q, const jvpattn_tensor *k, const jvpattn_tensor *v,
                const jvpattn_tensor *tq, const jvpattn_tensor *tk, const jvpattn_tensor *tv,
                const jvpattn_tensor *o, const jvpattn_tensor *to, float *lse, float *mu, float *li, void *stream) {
  FwdArgs a{};
  JVP_TRY(check_problem(p));
  if (is_empty(p) || p->len_q == 0) return JVPATTN_OK;  // nothing to write; pointers of empty tensors may be NULL
  JVP_TRY(build_fwd(p, q, k, v, tq, tk, tv, o, to, lse, mu, li, &a));
  DeviceInfo *d = nullptr;
  JVP_TRY(current_device(&d));
  a.status = d->status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  bool fast = p->kernels != JVPATTN_KERNELS_SIMT && sm100_fwd_supported(a);
  if (p->kernels == JVPATTN_KERNELS_TCGEN05 && !fast) return JVPATTN_EINVAL;
  if (fast) a.inject = g_inject_fwd.exchange(0);  // one-shot test hook
  return note_cuda(fast ? sm100_fwd(a, s) : simt_fwd(a, s));
}

size_t jvpattn_bwd_workspace_bytes(const jvpattn_problem *p) {
  if (check_problem(p) != JVPATTN_OK) return 0;
  return sm100_bwd_workspace_bytes(p->batch, p->heads, p->len_q, p->len_k, p->head_dim, p->stat_len);
}

int jvpattn_bwd(const jvpattn_problem *p, const jvpattn_tensor *q, const jvpattn_tensor *k, const jvpattn_tensor *v,
                const jvpattn_tensor *tq, const jvpattn_tensor *tk, const jvpattn_tensor *tv,
                const jvpattn_tensor *o, const jvpattn_tensor *to, const jvpattn_tensor *g_o, const jvpattn_tensor *g_to,
                const float *lse, const float *mu, const jvpattn_tensor *dq, const jvpattn_tensor *dk,
                const jvpattn_tensor *dv, const jvpattn_tensor *dtq, const jvpattn_tensor *dtk, const jvpattn_tensor *dtv,
                void *workspace, size_t workspace_bytes, void *stream) {
  BwdArgs a{};
  JVP_TRY(check_problem(p));
  if (is_empty(p)) return JVPATTN_OK;
  JVP_TRY(build_bwd(p, q, k, v, tq, tk, tv, o, to, g_o, g_to, lse, mu, dq, dk, dv, dtq, dtk, dtv, &a));
  size_t need = jvpattn_bwd_workspace_bytes(p);
  if (need > 0 && (!workspace || workspace_bytes < need)) return JVPATTN_EWORKSPACE;
  if (workspace && reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return JVPATTN_EALIGN;
  DeviceInfo *d = nullptr;
  JVP_TRY(current_device(&d));
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.status = d->status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  bool fast = p->kernels != JVPATTN_KERNELS_SIMT && sm100_bwd_supported(a);
  if (p->kernels == JVPATTN_KERNELS_TCGEN05 && !fast) return JVPATTN_EINVAL;
  return note_cuda(fast ? sm100_bwd(a, s) : simt_bwd(a, s));
}

// ------------------------------------------------------------------------------------------------
// Backward for callers that cannot allocate device memory.
//
// Some hosts of this library have no allocator to offer: a plug-in that only receives tensor pointers
// from its framework, a process whose memory pool has already claimed all of HBM, or a code region where
// calling cudaMalloc (or the framework's caching allocator) is forbidden.  jvpattn_bwd asks such a caller
// for a workspace it cannot produce.  This variant keeps the scratch (the two fp32 row-dot vectors,
// 2 * batch * heads * stat_len floats) in a fixed array inside the library image instead.
//
// The array lives in every CUDA context that loads the library (2 MiB per GPU, until the process exits).
// Host code cannot use the symbol's name as a pointer: the address is resolved per device with
// cudaGetSymbolAddress the first time the entry point is called with that device current, and cached.
// That first call therefore does set-up work beyond enqueueing kernels and should be made before any
// stream capture is started.
//
// All calls on a device share the one array and it keeps whatever the previous call left there.  Nothing
// in it has to start at zero (the row-dot kernel overwrites every element the later kernels read), but
// two calls that overlap on the GPU (different streams, no ordering between them) race on it; order them.
static __device__ __align__(256) float g_static_scratch[2 * JVPATTN_STATIC_SCRATCH_ROWS];

namespace {
struct StaticScratchSlot {
  int state = 0;  // 0 not resolved, 1 resolved, -1 failed
  void *ptr = nullptr;
};
StaticScratchSlot g_static_slots[kMaxDevices];
std::mutex g_static_mutex;
}  // namespace

int jvpattn_bwd_static(const jvpattn_problem *p, const jvpattn_tensor *q, const jvpattn_tensor *k, const jvpattn_tensor *v,
                       const jvpattn_tensor *tq, const jvpattn_tensor *tk, const jvpattn_tensor *tv,
                       const jvpattn_tensor *o, const jvpattn_tensor *to, const jvpattn_tensor *g_o,
                       const jvpattn_tensor *g_to, const float *lse, const float *mu, const jvpattn_tensor *dq,
                       const jvpattn_tensor *dk, const jvpattn_tensor *dv, const jvpattn_tensor *dtq,
                       const jvpattn_tensor *dtk, const jvpattn_tensor *dtv, void *stream) {
  JVP_TRY(check_problem(p));
  if (is_empty(p)) return JVPATTN_OK;
  const int64_t rows = (int64_t)p->batch * p->heads * p->stat_len;
  if (rows > JVPATTN_STATIC_SCRATCH_ROWS) return JVPATTN_ETOOLARGE;
  if (jvpattn_bwd_workspace_bytes(p) > sizeof(float) * 2 * JVPATTN_STATIC_SCRATCH_ROWS) return JVPATTN_ETOOLARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    note_cuda(e);
    return JVPATTN_EARCH;
  }
  void *scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticScratchSlot &slot = g_static_slots[dev];
    if (slot.state == 0) {
      void *ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_static_scratch);  // device address of the array in THIS device's context
      if (e != cudaSuccess || ptr == nullptr) {
        note_cuda(e);
        slot.state = -1;
      } else {
        slot.ptr = ptr;
        slot.state = 1;
      }
    }
    if (slot.state != 1) return JVPATTN_EARCH;
    scratch = slot.ptr;
  }
  return jvpattn_bwd(p, q, k, v, tq, tk, tv, o, to, g_o, g_to, lse, mu, dq, dk, dv, dtq, dtk, dtv, scratch,
                     sizeof(float) * 2 * JVPATTN_STATIC_SCRATCH_ROWS, stream);
}

}  // extern "C"
