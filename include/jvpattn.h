/*
 * jvpattn - C ABI of the B200 (sm_100a) flash-attention JVP kernels.
 *
 * The library replaces the three GPU entry points that the reference's autograd glue
 * (semicat/jvp_utils/functional.py) calls:
 *
 *   jvpattn_fwd   <- flash_attention_jvp_multihead_triton_kernel_wrapper
 *                    (semicat/jvp_utils/ryu_triton.py:295-422, called at functional.py:28-40)
 *   jvpattn_bwd   <- _flash_attn_backward of the tangent output
 *                    (semicat/jvp_utils/flash_jvp_backward.py:2293-2714, called at functional.py:131-149)
 *                    and _flash_attn_backward of the primal output
 *                    (semicat/jvp_utils/flash_attn_triton.py:974-1093, called at functional.py:192-205),
 *                    merged: either cotangent may be NULL.
 *
 * Conventions
 *   - plain C types only; every pointer is a CUDA device pointer owned by the caller, except where noted.
 *   - the library allocates no device memory; scratch is passed in (jvpattn_bwd_workspace_bytes).
 *   - kernels are enqueued on `stream` (a cudaStream_t cast to void*) of the CURRENT device; no host sync.
 *   - return value 0 on success, a negative JVPATTN_E* code otherwise; nothing is thrown.
 *   - there is no CPU path: without a usable sm_100 device every compute call returns JVPATTN_EARCH.
 */
#ifndef JVPATTN_H_
#define JVPATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define JVPATTN_ABI_VERSION 1

enum {
  JVPATTN_OK = 0,
  JVPATTN_EINVAL = -1,    /* NULL where a tensor is required, bad dims, bad dtype             */
  JVPATTN_ESTRIDE = -2,   /* innermost stride != 1                                            */
  JVPATTN_EALIGN = -3,    /* base pointer or a stride not 16-byte aligned                     */
  JVPATTN_EHEADDIM = -4,  /* head dim outside [16, 128] (ryu_triton.py:319-322, flash_jvp_backward.py:2318) */
  JVPATTN_ESTAT = -5,     /* row-statistic length not a multiple of 128 or < Lq (functional.py:124-125)     */
  JVPATTN_EWORKSPACE = -6,/* workspace NULL or smaller than jvpattn_bwd_workspace_bytes()     */
  JVPATTN_EARCH = -7,     /* no CUDA device, or the device is not sm_100                      */
  JVPATTN_ELAUNCH = -8,   /* the CUDA runtime refused a launch; see jvpattn_last_cuda_error() */
  JVPATTN_EDEVICE = -9,   /* jvpattn_stream_check: a bounded device-side wait ran out; see jvpattn_device_status() */
  JVPATTN_ETOOLARGE = -10 /* jvpattn_bwd_static: problem larger than the built-in scratch     */
};

enum { JVPATTN_BF16 = 0, JVPATTN_FP16 = 1 };

/* Selects the kernel family.  AUTO picks the tcgen05/TMA kernels whenever the shape allows and the
 * portable SIMT kernels otherwise; the other two force one family (the forced tcgen05 choice returns
 * JVPATTN_EINVAL for a shape it cannot run).  Used by the parity tests to check one family against
 * the other on the device. */
enum { JVPATTN_KERNELS_AUTO = 0, JVPATTN_KERNELS_SIMT = 1, JVPATTN_KERNELS_TCGEN05 = 2 };

/* A 4-D tensor indexed (batch, head, position, channel) with element strides; stride[3] must be 1.
 * The reference passes (B,H,S,D) views of (B,S,H,D)-contiguous memory (functional.py:324-326), so
 * stride[1] < stride[2] is the common case. */
typedef struct {
  void *ptr;
  int64_t stride[4];
} jvpattn_tensor;

typedef struct {
  int32_t batch, heads;
  int32_t len_q, len_k;
  int32_t head_dim;
  int32_t stat_len;  /* allocated row length of lse / mu / li: ceil(len_q/128)*128 (functional.py:57-59, 229-230) */
  int32_t dtype;     /* JVPATTN_BF16 or JVPATTN_FP16 for every jvpattn_tensor */
  int32_t kernels;   /* JVPATTN_KERNELS_* */
  float scale;       /* softmax scale; <= 0 selects 1/sqrt(head_dim) (ryu_triton.py:324-325) */
} jvpattn_problem;

/* Fused forward: O = softmax(scale QK^T) V together with its tangent Od along (tq, tk, tv), and the row
 * statistics lse = logsumexp(s) (the reference's M), mu = E_P[sd] (its MU); li (its LI, the softmax
 * denominator) is written only when non-NULL.  lse/mu/li are float32 [batch, heads, stat_len]; rows
 * >= len_q are not written.  o and to are written in place.
 * Primal-only form: with tq, tk, tv, to all NULL (mu may then be NULL too) the call is plain attention, O and lse
 * only.  It stands in for the F.scaled_dot_product_attention call of the reference's non-JVP branch
 * (semicat/net/duo.py:143-152); its backward is jvpattn_bwd with g_to = NULL.  Passing some but not all of the
 * four is JVPATTN_EINVAL. */
int jvpattn_fwd(const jvpattn_problem *p,
                const jvpattn_tensor *q, const jvpattn_tensor *k, const jvpattn_tensor *v,
                const jvpattn_tensor *tq, const jvpattn_tensor *tk, const jvpattn_tensor *tv,
                const jvpattn_tensor *o, const jvpattn_tensor *to,
                float *lse, float *mu, float *li, void *stream);

/* Bytes of scratch jvpattn_bwd needs for this problem: two float32 row vectors of batch * heads * stat_len
 * elements each (the row dot products rowsum(g_to o O) and rowsum(g_to o Od) + rowsum(g_o o O)), rounded up to
 * 256 bytes.  Returns 0 for an invalid problem. */
size_t jvpattn_bwd_workspace_bytes(const jvpattn_problem *p);

/* Backward: VJP of cotangents g_o (on O) and g_to (on Od) with respect to q, k, v, tq, tk, tv.
 * Either cotangent may be NULL (treated as zero) but not both.  dq, dk, dv are always written.
 * tq, tk, tv, to, mu, dtq, dtk, dtv are required when g_to is given; when it is NULL they are ignored
 * (may be NULL) and no tangent gradient is written.
 * `workspace` need not be initialised.
 * The call issues several kernels on `stream`; those of them that do not depend on each other run
 * concurrently (the kernels that write dk / dv beside the one that writes dq), so no output tensor may
 * overlap an input tensor or another output.  Work enqueued on the stream after the call sees all results. */
int jvpattn_bwd(const jvpattn_problem *p,
                const jvpattn_tensor *q, const jvpattn_tensor *k, const jvpattn_tensor *v,
                const jvpattn_tensor *tq, const jvpattn_tensor *tk, const jvpattn_tensor *tv,
                const jvpattn_tensor *o, const jvpattn_tensor *to,
                const jvpattn_tensor *g_o, const jvpattn_tensor *g_to,
                const float *lse, const float *mu,
                const jvpattn_tensor *dq, const jvpattn_tensor *dk, const jvpattn_tensor *dv,
                const jvpattn_tensor *dtq, const jvpattn_tensor *dtk, const jvpattn_tensor *dtv,
                void *workspace, size_t workspace_bytes, void *stream);

/* Caller-side helper (no counterpart in the reference's kernel wrappers; it replaces the pointwise chain in front
 * of them: the fp32 rotary embedding of q and k, semicat/net/duo.py:52-53, and the cast to bf16 in safe_sdpa_jvp,
 * semicat/jvp_utils/functional.py:318-321).  Rotates the two halves of the last axis of a strided (B, S, H, D)
 * view `x` (element strides sb, ss, sh; last stride 1) by the angles in `cos`, `sin` (fp32, (S, D/2) contiguous) and
 * writes a contiguous (B, S, H, D) tensor `y` of type `out_dtype`; `transpose` != 0 applies the transposed map (the
 * VJP).  fp32 products and sums are rounded separately, so the result is the fp32 formula rounded once.
 * dtype codes: JVPATTN_BF16, JVPATTN_FP16, JVPATTN_FP32.  D must be a multiple of 16. */
#define JVPATTN_FP32 2
int jvpattn_rotary_cast(const void *x, int64_t sb, int64_t ss, int64_t sh, int in_dtype, void *y, int out_dtype,
                        const float *cos, const float *sin, int batch, int len, int heads, int head_dim, int transpose,
                        void *stream);

/* jvpattn_rotary_cast for q, k and v of one projection in one launch: three (input view, output view) pairs of shape
 * (batch, len, heads, head_dim) with unit channel stride; pairs 0 and 1 are rotated (transpose as above), pair 2 is
 * copied (and cast).  in_strides / out_strides: element strides of (batch, position, head) for each pair, 3 x 3 values;
 * every pointer 16-byte aligned, every stride a multiple of 8 (else JVPATTN_EALIGN).  Forward: the three inputs are the
 * slices of the block's (batch, len, 3, heads, head_dim) projection, the outputs three contiguous tensors; backward
 * (transpose = 1): the inputs are the three gradients and the outputs the slices of the projection's gradient, which is
 * thereby written in place (semicat/net/duo.py:137-141).  Dtypes: JVPATTN_BF16 or JVPATTN_FP32 on either side. */
int jvpattn_rotary_qkv(const void *const in[3], const int64_t in_strides[9], int in_dtype, void *const out[3],
                       const int64_t out_strides[9], int out_dtype, const float *cos, const float *sin, int batch, int len,
                       int heads, int head_dim, int transpose, void *stream);

/* Caller-side helpers for the denoiser block around the attention (no counterpart among the reference's kernel wrappers;
 * they replace chains of PyTorch pointwise ops that, under torch.func.jvp, run as separate primal and tangent kernels):
 *   jvpattn_ln_modulate (+ jvpattn_ln_finalize)                 h = LayerNorm(x) * (1 + scale) + shift   (semicat/net/duo.py:128-135, 159)
 *   jvpattn_gated_residual, jvpattn_gated_residual_dual         z = x + mask * (gate * y)                (duo.py:157, 160)
 *   jvpattn_gelu_dual                                           the MLP's GELU                           (duo.py:118-123)
 * on (primal, tangent) pairs, with the VJPs of cotangents on both outputs.  x, y, masks, outputs and gradients are
 * contiguous (batch, len, channels) tensors, shift / scale / gate are (batch, channels) views whose rows are `*_stride`
 * elements apart, gamma / beta are fp32 (channels); every other tensor has the one element type `dtype` (JVPATTN_BF16 or
 * JVPATTN_FP32).
 *
 * jvpattn_ln_modulate: channels must be 256, 512, 768 or 1024 (else JVPATTN_EINVAL: the caller keeps its PyTorch ops).
 * `which`: 0 forward (y; also writes mean / rstd, fp32 (batch * len)), 1 forward of the tangent (ty from tx and the
 * tangents of the modulation; NULL tangents are zeros), 2 VJP of a cotangent `g` on y (writes dx), 3 VJP of a cotangent on
 * ty (writes dx and dtx).  The VJPs ADD per-sample column sums into `sums` (fp32; which = 2: (2, batch, channels) = sum_s g n,
 * sum_s g with n the normalised row; which = 3: (3, batch, channels) = sum_s g n, sum_s g, sum_s g nd with nd the tangent of n),
 * which the caller zeroes beforehand and hands to jvpattn_ln_finalize.  `exact` bit 0 selects the VJP of the LayerNorm
 * tangent with respect to x: 0 reproduces PyTorch,
 * whose forward-mode formula for native_layer_norm treats the saved mean / rstd as constants when it is differentiated
 * again; 1 includes their dependence on x.  Bit 1 (which = 3 only): add to what dx holds instead of overwriting it, so that
 * the two backward kernels of one (primal, tangent) pair leave their sum. */
int jvpattn_ln_modulate(int which, const void *x, const void *tx, const float *gamma, const float *beta, const void *shift,
                        const void *scale, const void *tshift, const void *tscale, int64_t mod_stride, int64_t tmod_stride,
                        float *mean, float *rstd, void *out, const void *g, void *dx, void *dtx, float *sums, int batch, int len,
                        int channels, float eps, int exact, int dtype, void *stream);
/* Dropout keep mask generated inside the gated-residual kernels instead of read from `mask` (used when `mask` is NULL):
 * element e of the call is kept with probability 1 - p and scaled by 1 / (1 - p); the decision is a counter-based hash
 * (Philox-4x32-10) of (*seed, call, e / 8), so every kernel given the same three values sees the same mask - forward,
 * tangent and backward of one call of one step.  `seed` is read from DEVICE memory at run time: draw it once per step
 * (inside the captured graph, if there is one) and number the calls of the step with `call`. */
typedef struct jvpattn_dropout {
  const uint64_t *seed;
  uint32_t call;
  float p;
} jvpattn_dropout;

/* z = x + m gate y for the passes without a tangent (m = `mask`, or generated from `drop`, or all ones); gate: (batch,
 * channels) rows `gate_stride` elements apart; channels a multiple of 8.  Its backward is jvpattn_gated_residual_dual
 * (which = 1) with gtz = NULL. */
int jvpattn_gated_residual(const void *x, const void *y, const void *gate, const void *mask, int64_t gate_stride, void *z,
                           int batch, int len, int channels, int dtype, const jvpattn_dropout *drop, void *stream);

/* Vocabulary-side head of the flow-map step (no counterpart among the reference's kernel wrappers; it replaces the softmax
 * over the vocabulary and the pointwise chain around it in semicat/models/semicat.py:210-229 and its forward-mode tangent,
 * :153-157):   xst = x + dt (softmax(logits) - x),   dv = ddt (p - x) + dt p o (tlogits - sum(p tlogits)).
 * logits / tlogits: (batch, rows_per_sample, vocab) of `dtype` (JVPATTN_BF16 or JVPATTN_FP32) with rows `ld_*` elements
 * apart; x, out, g: fp32 contiguous; dt, ddt: fp32 (batch); lse: fp32 (batch * rows_per_sample), written by which = 0
 * and read by the others.  which: 0 forward (out = xst), 1 forward of the tangent (out = dv), 2 VJP of a cotangent g on
 * xst (writes dlogits), 3 VJP of a cotangent g on dv (writes dlogits and dtlogits); gradients are contiguous, in `dtype`.
 * x, dt and ddt are data of the step (no gradient is formed for them).  A row pair must fit 200 KB of shared memory
 * (vocab <= 51200 for bf16, 25600 for fp32), else JVPATTN_EINVAL. */
int jvpattn_flow_map_head(int which, const void *logits, const void *tlogits, int64_t ld_logits, int64_t ld_tlogits, const float *x,
                          const float *dt, const float *ddt, float *lse, float *out, const float *g, void *dlogits,
                          void *dtlogits, int batch, int rows_per_sample, int vocab, int dtype, void *stream);

/* GELU (tanh form) of the block's MLP on a (primal, tangent) pair (semicat/net/duo.py:118-123), n contiguous elements of
 * `dtype` (n a multiple of 8, 16-byte aligned pointers).
 * mode 0: out = gelu(h).
 * mode 1: out = gelu'(h) * v - the forward-mode tangent (v = tangent of h) and the VJP of either output with respect to
 *         its own input (v = cotangent).
 * mode 2: out = gelu'(h) * v and out2 = gelu''(h) * w * v - the VJP of the tangent output (v = its cotangent, w = the
 *         tangent of h) with respect to the tangent (out) and to h (out2).
 * mode 3: out = gelu(h) and out2 = gelu'(h) * v - primal and tangent in one pass.
 * mode 4: out = gelu'(h) * v + gelu''(h) * w * u and out2 = gelu'(h) * u - both cotangents in one pass (v on the primal
 *         output, u on the tangent output, w = the tangent of h): out = gradient of h, out2 = gradient of the tangent. */
int jvpattn_gelu_dual(int mode, const void *h, const void *v, const void *w, const void *u, void *out, void *out2, int64_t n,
                      int dtype, void *stream);

/* Gated residual on a (primal, tangent) pair in one pass each way (the merged form of jvpattn_gated_residual):
 * which 0: z = x + m gate y and tz = tx + m (gate ty + tgate y)            (tx, ty, tgate, mask may be NULL)
 * which 1: from cotangents gz on z and gtz on tz (either may be NULL): d_y = m (gate gz + tgate gtz), d_ty = m gate gtz,
 *          sums[0][b] += sum_s m (y gz + ty gtz) (gradient of gate), sums[1][b] += sum_s m y gtz (gradient of tgate);
 *          sums: fp32 (2, batch, channels), zeroed by the caller.  The skip gradients are gz and gtz themselves.
 * channels: a multiple of 8, at most 1024. */
int jvpattn_gated_residual_dual(int which, const void *x, const void *tx, const void *y, const void *ty, const void *gate,
                                const void *tgate, const void *mask, int64_t gate_stride, int64_t tgate_stride, void *z, void *tz,
                                const void *gz, const void *gtz, void *d_y, void *d_ty, float *sums, int batch, int len,
                                int channels, int dtype, const jvpattn_dropout *drop, void *stream);

/* Turns the column sums that jvpattn_ln_modulate's backward kernels leave (sums_y: which = 2, (2, batch, channels);
 * sums_ty: which = 3, (3, batch, channels); either may be NULL) into the gradients of shift, scale, their tangents
 * ((batch, channels) contiguous in `dtype`; NULL = not wanted) and of the LayerNorm weight and bias (fp32 (channels),
 * zeroed by the caller: the kernel adds to them), in one launch. */
int jvpattn_ln_finalize(const float *sums_y, const float *sums_ty, const float *gamma, const float *beta, const void *scale,
                        const void *tscale, int64_t mod_stride, int64_t tmod_stride, void *d_shift, void *d_scale, void *d_tshift,
                        void *d_tscale, float *d_gamma, float *d_beta, int batch, int channels, int dtype, void *stream);

/* Vocabulary-side ends of the flow-map training step with nothing of size (rows, vocab) materialised in fp32
 * (no counterpart among the reference's kernel wrappers; replaces the PyTorch passes of semicat/models/semicat.py:70-85,
 * 89-110, 112-167 with sd_type "lag", 210-229).  rows = batch * rows_per_sample; row r belongs to sample r / rows_per_sample.
 *   x0      fp32 noise, row pitch ldx elements;   ids  int64 (rows) token ids;   s, t  fp32 (batch) times
 *   logits, tlogits, target_logits   `dtype` (JVPATTN_BF16 or JVPATTN_FP32), row pitch ld (multiple of 8, >= vocab rounded
 *            up to 8; the columns from vocab on are ignored), 16-byte aligned
 *   out, out2   `dtype`, row pitch ldo (same rule); columns from vocab on are written as zeros
 *   lse (rows), stats (rows, 4), loss (rows)   fp32;   g   fp32 scalar in device memory: cotangent of the MEAN of `loss`
 * op 0  out = (1 - t) x0 + t onehot(ids)                                            (the interpolated input, :70-85)
 * op 1  out = xs + dt (softmax(logits) - xs), xs = (1 - s) x0 + s onehot(ids), dt = (t - s) / (1 - s + 1e-8); writes lse
 * op 2  loss = cross-entropy(logits, ids) with label smoothing eps; writes lse       (:107-111)
 * op 3  out = g / rows * d loss / d logits                                           (reads lse)
 * op 4  loss = sum_v ((1 - t) dv - softmax(target_logits) + xst)^2 with xst as in op 1 and
 *       dv = ddt (p - xs) + dt p o (tlogits - sum(p tlogits)), ddt = 1 / (1 - s + 1e-8); reads lse (op 1), writes stats
 * op 5  out, out2 = g / rows * d loss / d (logits, tlogits)                          (reads lse and stats) */
int jvpattn_vocab_op(int op, const void *logits, const void *tlogits, const void *target_logits, int64_t ld, const float *x0,
                     int64_t ldx, const int64_t *ids, const float *s, const float *t, float *lse, float *stats, float *loss,
                     const float *g, void *out, void *out2, int64_t ldo, float eps, int batch, int rows_per_sample, int vocab,
                     int dtype, void *stream);

/* Same backward for callers that have no way to allocate device memory (no counterpart in the reference,
 * whose wrappers allocate freely through torch).  Takes no workspace: the scratch lives in a fixed
 * 2 MiB array inside the library image, present on every GPU that loads the library until the process
 * exits.  Limit: batch * heads * stat_len <= JVPATTN_STATIC_SCRATCH_ROWS, otherwise JVPATTN_ETOOLARGE
 * and nothing is launched.  The call itself allocates nothing.  The first call on each device resolves
 * the array's device address (cudaGetSymbolAddress) and should come before any stream capture.  All calls
 * on a device share the array: calls that overlap on the GPU race and must be ordered by the caller. */
#define JVPATTN_STATIC_SCRATCH_ROWS 262144
int jvpattn_bwd_static(const jvpattn_problem *p,
                       const jvpattn_tensor *q, const jvpattn_tensor *k, const jvpattn_tensor *v,
                       const jvpattn_tensor *tq, const jvpattn_tensor *tk, const jvpattn_tensor *tv,
                       const jvpattn_tensor *o, const jvpattn_tensor *to,
                       const jvpattn_tensor *g_o, const jvpattn_tensor *g_to,
                       const float *lse, const float *mu,
                       const jvpattn_tensor *dq, const jvpattn_tensor *dk, const jvpattn_tensor *dv,
                       const jvpattn_tensor *dtq, const jvpattn_tensor *dtk, const jvpattn_tensor *dtv,
                       void *stream);

/* Which kernel family AUTO resolves to for this problem (JVPATTN_KERNELS_SIMT or _TCGEN05), for the
 * forward (which = 0) or the backward (which = 1); negative error code for an invalid problem. */
int jvpattn_selected_kernels(const jvpattn_problem *p, int which);

/* Number of kernels this library has launched in the calling process (all threads). */
uint64_t jvpattn_launch_count(void);

/* Optional per-kernel timing for measurement harnesses (no counterpart in the reference, which relies on
 * triton.testing.do_bench around whole calls, ryu_triton.py:958-1007).  Between _begin and _end every
 * launch is bracketed by CUDA events on its stream; _end synchronises the device and returns, per kernel
 * id in [0, JVPATTN_NUM_KERNELS), the summed device time in milliseconds and the launch count. */
#define JVPATTN_NUM_KERNELS 9
int jvpattn_profile_begin(void);
int jvpattn_profile_end(double *total_ms, uint64_t *launches);
const char *jvpattn_kernel_name(int id);

/* Synchronises the current device and returns the device-side status word: 0 if no bounded wait has
 * run out since the last call, else a code identifying the wait that gave up (101..107 forward, 201..216
 * backward).  Clears the word.  Every wait inside the kernels is bounded (about two seconds): a kernel whose
 * wait runs out stops computing, leaves through its normal teardown and leaves its outputs unwritten or partial;
 * the context stays usable. */
int jvpattn_device_status(void);

/* Waits for the work enqueued on `stream` and returns JVPATTN_EDEVICE if a device-side wait has run out since the
 * status word was last cleared (the word is left in place for jvpattn_device_status), else JVPATTN_OK.  The
 * reference has no counterpart: its Triton kernels contain no waits that could fail. */
int jvpattn_stream_check(void *stream);

/* Test hooks for the failure path (no counterpart in the reference; not for production use).
 *   JVPATTN_DEBUG_WAIT_CYCLES     value = budget of every device-side wait in clock cycles for kernels launched from
 *                                 now on; value <= 0 restores the default (about two seconds).
 *   JVPATTN_DEBUG_STALL_NEXT_FWD  value != 0: in the next tcgen05 forward launch (only that one) the barrier of every
 *                                 CTA's first key tile expects bytes that never arrive, so the waits behind it run out:
 *                                 the kernel must end by itself, report a 10x status code and leave the device usable. */
enum { JVPATTN_DEBUG_WAIT_CYCLES = 0, JVPATTN_DEBUG_STALL_NEXT_FWD = 1 };
int jvpattn_debug_set(int knob, long long value);

const char *jvpattn_strerror(int code);
const char *jvpattn_last_cuda_error(void); /* text of the last CUDA runtime error seen by this thread */
int jvpattn_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* JVPATTN_H_ */
