/* ane_cuda.h -- C ABI of libane_cuda: the maderix/ANE per-layer non-matmul operator set as
 * hand-written CUDA kernels for NVIDIA B200 (sm_100a).
 *
 * The boundary follows the one C ABI the reference has, bridge/ane_bridge.h:16-94: opaque
 * handles, int status returns, byte-count reads and writes of device-visible buffers, explicit
 * free, no C++ types.  Three groups of entry points:
 *
 *   1. lifecycle and device buffers        (the ane_bridge_init / write_input / read_output
 *                                           / free analogue)
 *   2. host-buffer entry points            (a) drop-ins with the argument order and overwrite /
 *                                           accumulate behaviour of the `static` functions of
 *                                           training/stories_cpu_ops.h and
 *                                           training/training_dynamic/cpu_ops.h; (b) batched,
 *                                           any-dtype, fused forms.  Both stage host <-> device
 *                                           and are PCIe-bound
 *   3. device-resident operators (`_dev`)  asynchronous on a caller-given CUDA stream; these
 *                                           are what a GPU training loop calls and what the
 *                                           benchmark times
 *
 * Tensor layout everywhere: channel-first, batched as [B][C][S]; element (b, c, t) lives at
 * (b*C + c)*S + t (training/stories_cpu_ops.h:10,117).  S is the contiguous axis.
 *
 * There is no CPU fallback: every operator runs on the GPU or returns an error.
 * Threading: one host thread per device at a time (the reference's operators are likewise
 * never re-entered concurrently, training/training_dynamic/train.m:727-749).  Which thread that is
 * may change between calls; the text behind ane_cuda_last_error() is kept per thread.
 */
#ifndef ANE_CUDA_H
#define ANE_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ANE_CUDA_VERSION 100

/* ---- status codes (0 = success, negative = failure; ane_cuda_last_error() has the text) */
#define ANE_CUDA_OK              0
#define ANE_CUDA_ERR_INVALID    (-1)  /* bad argument: null pointer, non-positive size, misaligned ... */
#define ANE_CUDA_ERR_CUDA       (-2)  /* a CUDA runtime call failed */
#define ANE_CUDA_ERR_NOT_INIT   (-3)  /* ane_cuda_init() has not succeeded on this process */
#define ANE_CUDA_ERR_NOMEM      (-4)  /* device or pinned-host allocation failed */
#define ANE_CUDA_ERR_UNSUPPORTED (-5) /* shape outside what the kernels cover (documented per op) */
#define ANE_CUDA_ERR_TIMEOUT    (-6)  /* a bounded device-side wait gave up (status word has details) */

/* ---- element types of activation tensors (math is always fp32 inside the kernels) */
typedef enum { ANE_F32 = 0, ANE_BF16 = 1, ANE_F16 = 2 } ane_dtype;
/* ---- token id types: the reference uses uint16_t (stories_cpu_ops.h:112), Qwen3's vocabulary
 *      of 151936 needs int32 */
typedef enum { ANE_ID_U16 = 0, ANE_ID_I32 = 1 } ane_idtype;

/* ---- flags */
#define ANE_NORM_BWD_REFERENCE 0u /* dx = w*rrms*(dy - x*coef): what stories_cpu_ops.h:42-46 computes */
#define ANE_NORM_BWD_EXACT     1u /* dx = rrms*(w*dy - x*coef): analytic form, ane_rmsnorm_bwd.h:56,70-74 */
#define ANE_ROPE_FORWARD       0u
#define ANE_ROPE_INVERSE       1u /* the backward rotation of training_dynamic/cpu_ops.h:168-184 */
#define ANE_ADAM_STORIES       0u /* w -= lr*mh/(sqrt(vh)+eps)                 stories_cpu_ops.h:55-63 */
#define ANE_ADAM_DYNAMIC       1u /* w -= lr*(mh/(sqrt(vh)+eps) + wd*w)        training_dynamic/cpu_ops.h:56-64 */
#define ANE_OOR_SKIP           0u /* out-of-range id: leave the column / row untouched (stories_cpu_ops.h:115,126) */
#define ANE_OOR_ZERO           2u /* out-of-range id: write zeros instead */

/* AdamState, laid out as in training/stories_config.h:56-59 and training_dynamic/config.h:46. */
typedef struct { float *m, *v; size_t n; } AdamState;

/* Device-side status words written by the kernels (ane_cuda_poll_status copies them out). */
typedef struct {
    int32_t oor_ids;      /* token / target ids outside [0, vocab) seen since the last reset */
    int32_t nonfinite;    /* per-token losses that were not finite */
    int32_t wait_giveups; /* bounded device-side waits that ran out */
    int32_t reserved;
} ane_cuda_status;

typedef struct ANECudaBuf ANECudaBuf; /* opaque device buffer, the IOSurface analogue (ane_bridge.h:16) */

/* =====================================================================================
 * 1. Lifecycle and buffers                      replaces bridge/ane_bridge.h:20,54-68
 * ===================================================================================== */
/* Select `device`, create the library's context on it.  Idempotent per device, like
 * ane_bridge_init (bridge/ane_bridge.m:34).  Returns ANE_CUDA_OK or a negative code. */
int ane_cuda_init(int device);
void ane_cuda_shutdown(void);
int ane_cuda_version(void);
int ane_cuda_device_count(void);
const char *ane_cuda_last_error(void);
/* Number of this library's kernels launched since the last reset (cf. the compile counter of
 * ane_bridge.h:65-68). */
long long ane_cuda_launch_count(void);
void ane_cuda_reset_launch_count(void);

/* Kernel-selection knobs for benchmarking (tile shapes; every setting computes the same result
 * up to the summation order of dw).  Unknown names are stored and ignored. */
int ane_cuda_set_tuning(const char *name, int value);
/* Back to the built-in choice for one knob (NULL: for all of them). */
int ane_cuda_clear_tuning(const char *name);
/* One knob is a debugging aid rather than a kernel choice: "check_extents" = 1 makes every device-resident operator check,
 * before it launches anything, that each device range it will touch lies inside the allocation that holds the pointer
 * (the driver knows every allocation's extent); a buffer too small for the given shape returns ANE_CUDA_ERR_INVALID with
 * the argument's name.  One driver call per pointer, so it is off by default. */

ANECudaBuf *ane_cuda_alloc(size_t bytes);                       /* NULL on failure */
int ane_cuda_write(ANECudaBuf *buf, size_t offset, const void *host, size_t bytes);  /* ane_bridge_write_input */
int ane_cuda_read(ANECudaBuf *buf, size_t offset, void *host, size_t bytes);         /* ane_bridge_read_output */
void *ane_cuda_devptr(ANECudaBuf *buf);
size_t ane_cuda_bufsize(ANECudaBuf *buf);
void ane_cuda_free(ANECudaBuf *buf);                            /* ane_bridge_free */
/* Page-locked host memory; the drop-ins of group 2 copy asynchronously from / to it. */
void *ane_cuda_host_alloc(size_t bytes);
void ane_cuda_host_free(void *p);
int ane_cuda_sync(void *stream);
/* Clears `bytes` bytes of device memory on the stream (the memset of the accumulated gradients, train.m:874-877). */
int ane_cuda_zero_dev(void *stream, void *dev, size_t bytes);
/* Copy between device ranges on the stream; either side may be another GPU's memory mapped into this process (the copy
 * engines move it over NVLink, no SM is used -- what the gradient push of the data-parallel step relies on). */
int ane_cuda_copy_dev(void *stream, void *dst, const void *src, size_t bytes);
/* Copy the device status words to *out and optionally clear them. */
int ane_cuda_poll_status(ane_cuda_status *out, int reset);
/* Bytes of library-owned scratch currently held on the device (grow-only cache). */
size_t ane_cuda_workspace_bytes(void);
/* Library-owned device memory and CUDA graphs.  Operators keep two kinds of device memory between calls: the scratch
 * range (dw partials, sort buffers, per-token losses) and cached RoPE cos/sin tables, one per (head width, S, base,
 * first position), at most 64.  The rule: an address that an operator has used is never freed, moved or refilled with
 * other contents before ane_cuda_shutdown / ane_cuda_release_caches -- when the scratch must grow, a new range is
 * allocated and the old one is kept -- so work already enqueued and graphs already captured stay valid whatever is
 * called later.  What a capture needs must exist BEFORE the capture: run every operator once with the arguments to be
 * captured (or call ane_cuda_reserve_workspace), because an allocation inside a capture is refused
 * (ANE_CUDA_ERR_NOMEM for scratch, ANE_CUDA_ERR_UNSUPPORTED for a missing RoPE table; ane_cuda_rope_dev alone falls
 * back to evaluating cos/sin in the kernel).  ane_cuda_freeze(1) turns every later growth or new table into that
 * same refusal, outside captures too: a loop that must not allocate calls it after warm-up; ane_cuda_freeze(0) lifts it.
 * A table filled on one stream and used on another is ordered by an event. */
int ane_cuda_reserve_workspace(size_t bytes);
int ane_cuda_freeze(int on);
/* Frees the cached RoPE tables and the scratch ranges that were replaced by larger ones, after a device-wide
 * synchronisation.  Only when no captured graph that used them will be launched again. */
int ane_cuda_release_caches(void);

/* =====================================================================================
 * 2. Host-buffer entry points
 * ===================================================================================== */
/* 2a. Reference signatures: fp32, one sequence, the reference's literals (eps 1e-5, base 1e4). */
/* training/stories_cpu_ops.h:6 and training_dynamic/cpu_ops.h:7 -- rmsnorm(out,x,w,d,S) */
int ane_cuda_rmsnorm(float *out, const float *x, const float *w, int d, int S);
/* stories_cpu_ops.h:23 / cpu_ops.h:24 -- dx is overwritten, dw is accumulated into */
int ane_cuda_rmsnorm_bwd(float *dx, float *dw, const float *dy, const float *x, const float *w, int d, int S);
/* stories_cpu_ops.h:55 */
int ane_cuda_adam_update(float *w, const float *g, AdamState *s, int t, float lr, float b1, float b2, float eps);
/* training_dynamic/cpu_ops.h:56 (decoupled weight decay inside the lr bracket) */
int ane_cuda_adam_update_wd(float *w, const float *g, AdamState *s, int t, float lr, float b1, float b2,
                            float eps, float wd);
/* stories_cpu_ops.h:71 / cpu_ops.h:68 -- returns the mean loss through *loss; an out-of-range
 * target behaves as stories_cpu_ops.h:94-103 (column keeps the plain softmax, no loss term) */
int ane_cuda_cross_entropy_loss(float *loss, float *dlogits, const float *logits, const uint16_t *targets,
                                int V, int S);
/* stories_cpu_ops.h:112 / cpu_ops.h:150 -- `vocab` is the reference's compile-time VOCAB */
int ane_cuda_embed_lookup(float *x, const float *embed, const uint16_t *tokens, int dim, int seq, int vocab);
/* stories_cpu_ops.h:123 / cpu_ops.h:158 -- d_embed [vocab, dim] is accumulated into */
int ane_cuda_embed_backward(float *d_embed, const float *dx, const uint16_t *tokens, int dim, int seq, int vocab);
/* training_dynamic/cpu_ops.h:168 -- in place, base 10000 */
int ane_cuda_rope_backward_inplace(float *dx, int seq, int dim, int hd);
/* the inline blocks of training_dynamic/train.m: :460 residual, :537-554 SwiGLU backward */
int ane_cuda_residual(float *out, const float *x, const float *f, float alpha, size_t n);
int ane_cuda_swiglu(float *out, const float *h1, const float *h3, size_t n);
int ane_cuda_swiglu_bwd(float *dh1, float *dh3, const float *h1, const float *h3, const float *dsilu, size_t n);

/* 2b. Batched, any dtype, fused forms: the same operators as group 3 with activations in HOST
 * memory ([B][C][S], dtype elements; w / dw fp32).  The batch is cut into chunks that flow
 * through a three-stream pipeline (upload, kernel, download), so both PCIe directions overlap
 * the kernels when the buffers are page-locked (ane_cuda_host_alloc).  They block until the
 * results are in host memory.  Reference call sites as for the `_dev` forms below. */
int ane_cuda_rmsnorm_host(ane_dtype dtype, int B, int C, int S, void *out, const void *x, const float *w, float eps);
int ane_cuda_rmsnorm_bwd_host(ane_dtype dtype, int B, int C, int S, void *dx, float *dw, const void *dy,
                              const void *x, const float *w, const void *add, float eps, unsigned flags);
int ane_cuda_residual_host(ane_dtype dtype, size_t n, void *out, const void *x, const void *f, float alpha);
int ane_cuda_residual_rmsnorm_host(ane_dtype dtype, int B, int C, int S, void *x2, void *x2norm, const void *x,
                                   const void *f, const float *w, float alpha, float eps);
int ane_cuda_swiglu_host(ane_dtype dtype, size_t n, void *out, const void *h1, const void *h3);
int ane_cuda_swiglu_bwd_host(ane_dtype dtype, size_t n, void *dh1, void *dh3, const void *h1, const void *h3,
                             const void *dsilu);
int ane_cuda_rope_host(ane_dtype dtype, int B, int C, int S, int hd, void *out, const void *x, float base, int pos0,
                       unsigned flags);
int ane_cuda_qknorm_rope_host(ane_dtype dtype, int B, int heads, int hd, int S, void *out, const void *x,
                              const float *w, float eps, float base, int pos0);
int ane_cuda_rope_qknorm_bwd_host(ane_dtype dtype, int B, int heads, int hd, int S, void *dx, float *dw,
                                  const void *dy, const void *x, const float *w, float eps, float base, int pos0,
                                  unsigned flags);

/* =====================================================================================
 * 3. Device-resident operators.  `stream` is a cudaStream_t (NULL = default stream).
 *    All pointers are device pointers.  Weights (w, dw) and optimizer state are fp32;
 *    activations have `dtype`.  Vectorised paths need 16-byte aligned pointers and S a
 *    multiple of 16/sizeof(element); other shapes take a slower scalar path.
 * ===================================================================================== */
/* a1: out = (x * rrms) * w[c], rrms = 1/sqrt(mean_c x^2 + eps)         stories_cpu_ops.h:6-21 */
int ane_cuda_rmsnorm_dev(void *stream, ane_dtype dtype, int B, int C, int S,
                         void *out, const void *x, const float *w, float eps);
/* a2 (+a3 backward add): dx = rmsnorm_bwd(dy, x, w) [+ add] ; dw[c] += sum_tokens dy*x*rrms
 * (deterministic: per-block partials summed in a fixed order).  add may be NULL.
 * stories_cpu_ops.h:23-53 ; the add is training_dynamic/train.m:590,721 */
int ane_cuda_rmsnorm_bwd_dev(void *stream, ane_dtype dtype, int B, int C, int S,
                             void *dx, float *dw, const void *dy, const void *x, const float *w,
                             const void *add, float eps, unsigned flags);
/* Same operator and arguments as ane_cuda_rmsnorm_bwd_dev, for callers that must not cause a
 * device allocation -- e.g. a process whose framework has reserved the whole GPU for its own
 * memory pool, so that a cudaMalloc from this library would fail or fragment the pool, or a
 * latency-critical loop that cannot take cudaMalloc's device-wide synchronisation.  It has no
 * counterpart in the reference (whose rmsnorm_bwd mallocs its scratch on every call,
 * stories_cpu_ops.h:24-25).  The dw partials live in a fixed 2.3 MiB array inside the library
 * image (held on every GPU that loads the library until the process exits), so:
 *   - C must be <= 2048 (ANE_CUDA_ERR_UNSUPPORTED otherwise; B and S are not limited);
 *   - it does not need ane_cuda_init(), and calls no cudaMalloc / cudaFree or any allocating
 *     library routine; the caller passes inputs and outputs on the CURRENT device;
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress) -- make that first call before any stream capture, and make it at
 *     start-up, BEFORE a framework takes the rest of the device for its pool: with CUDA's lazy
 *     module loading the library image that contains the array is placed in device memory when
 *     one of its kernels is first used, so that first call may itself need 2.3 MiB of free memory;
 *   - all calls share the one array: calls that may overlap on the GPU (different streams,
 *     or other threads) race on it.  Keep them on one stream, or order them with events.
 * Results: the same operator as ane_cuda_rmsnorm_bwd_dev within fp32 rounding -- the two entry points
 * may run different kernels, whose per-token sums and dw partials are added in different (each
 * fixed) orders; a call with the same arguments gives the same bits every time. */
int ane_cuda_rmsnorm_bwd_static_dev(void *stream, ane_dtype dtype, int B, int C, int S,
                                    void *dx, float *dw, const void *dy, const void *x, const float *w,
                                    const void *add, float eps, unsigned flags);
/* a3: out = f*alpha + x (flat, n elements)                            train.m:460, mil_dynamic.h:279-283 */
int ane_cuda_residual_dev(void *stream, ane_dtype dtype, size_t n, void *out, const void *x, const void *f,
                          float alpha);
/* out = alpha * x                                                      train.m:497,523,595 */
int ane_cuda_scale_dev(void *stream, ane_dtype dtype, size_t n, void *out, const void *x, float alpha);
/* a3+a1 fused: x2 = f*alpha + x ; x2norm = rmsnorm(x2)                 train.m:460-461 */
int ane_cuda_residual_rmsnorm_dev(void *stream, ane_dtype dtype, int B, int C, int S,
                                  void *x2, void *x2norm, const void *x, const void *f, const float *w,
                                  float alpha, float eps);
/* a4: out = h1*sigmoid(h1)*h3                                          forward.h:101,149-151
 * The sigmoid of a4 / a5 comes from the hardware's exp2 and reciprocal approximations (relative error below 1e-6; values
 * under 2^-126, i.e. h1 < -87.3, become zero); tuning knob "swiglu_exact" = 1 selects expf and an IEEE division. */
int ane_cuda_swiglu_dev(void *stream, ane_dtype dtype, size_t n, void *out, const void *h1, const void *h3);
/* a5: dh1, dh3 from h1, h3, dsilu in one pass                          train.m:537-554 */
int ane_cuda_swiglu_bwd_dev(void *stream, ane_dtype dtype, size_t n, void *dh1, void *dh3,
                            const void *h1, const void *h3, const void *dsilu);
/* a6/a7: rotate interleaved channel pairs (2i, 2i+1) of every head by theta = (pos0+t)*base^(-2i/hd);
 * flags = ANE_ROPE_FORWARD or ANE_ROPE_INVERSE; out may equal x (in place).
 * cpu_ops.h:168-184, forward.h:55-70 */
int ane_cuda_rope_dev(void *stream, ane_dtype dtype, int B, int C, int S, int hd,
                      void *out, const void *x, float base, int pos0, unsigned flags);
/* a8: per-head RMSNorm over the hd channels of each head, weight w[hd] shared by the heads. */
int ane_cuda_qknorm_dev(void *stream, ane_dtype dtype, int B, int heads, int hd, int S,
                        void *out, const void *x, const float *w, float eps);
int ane_cuda_qknorm_bwd_dev(void *stream, ane_dtype dtype, int B, int heads, int hd, int S,
                            void *dx, float *dw, const void *dy, const void *x, const float *w,
                            float eps, unsigned flags);
/* a8+a6 fused: out = rope(qknorm(x)) */
int ane_cuda_qknorm_rope_dev(void *stream, ane_dtype dtype, int B, int heads, int hd, int S,
                             void *out, const void *x, const float *w, float eps, float base, int pos0);
/* a7+a8 fused: dx = qknorm_bwd(rope^-1(dy), x, w) ; dw[hd] += ... */
int ane_cuda_rope_qknorm_bwd_dev(void *stream, ane_dtype dtype, int B, int heads, int hd, int S,
                                 void *dx, float *dw, const void *dy, const void *x, const float *w,
                                 float eps, float base, int pos0, unsigned flags);
/* Q and K of one layer in one call: the two operators above applied to q [B][heads_q*hd][S] with wq and to k
 * [B][heads_k*hd][S] with wk.  The outputs (and dq, dk) carry the bits of the two separate calls; dwq / dwk are the same
 * sums added in another fixed order (bit-stable from call to call).  For head widths 64 and 128 with 16-byte aligned rows
 * the two launches run at the same time, each on its share of the GPU (heads_q : heads_k), K on a stream of the library
 * that is forked from and joined to the caller's stream inside the call (also under stream capture); other shapes, or knob
 * "qk_pair" = 0, make the two calls one after the other.  Same positions (pos0) and head width for both, as in a
 * transformer layer (no counterpart in the reference, which has no QK-norm: the RoPE of Q and K of a layer is one loop
 * there, training/training_dynamic/cpu_ops.h:168-184 called for dq and dk at train.m:659-660). */
int ane_cuda_qknorm_rope_pair_dev(void *stream, ane_dtype dtype, int B, int heads_q, int heads_k, int hd, int S,
                                  void *out_q, void *out_k, const void *q, const void *k, const float *wq,
                                  const float *wk, float eps, float base, int pos0);
int ane_cuda_rope_qknorm_bwd_pair_dev(void *stream, ane_dtype dtype, int B, int heads_q, int heads_k, int hd, int S,
                                      void *dq, void *dk, float *dwq, float *dwk, const void *dyq, const void *dyk,
                                      const void *q, const void *k, const float *wq, const float *wk, float eps,
                                      float base, int pos0, unsigned flags);
/* a9: x[b][d][t] = table[tok[b][t]][d] (bit-exact copy; table has the same dtype as x).
 * flags: ANE_OOR_SKIP (default) or ANE_OOR_ZERO.  stories_cpu_ops.h:112-120 */
int ane_cuda_embed_lookup_dev(void *stream, ane_dtype dtype, ane_idtype idtype, int B, int D, int S,
                              void *x, const void *table, const void *tokens, int vocab, unsigned flags);
/* a10: d_embed[tok[b][t]][d] += dx[b][d][t], fp32 accumulate in increasing (b, t) order per row;
 * run-to-run bit-identical (sort by id, then one writer per row).  stories_cpu_ops.h:123-131 */
int ane_cuda_embed_backward_dev(void *stream, ane_dtype dtype, ane_idtype idtype, int B, int D, int S,
                                float *d_embed, const void *dx, const void *tokens, int vocab);
/* a11: per token softmax over V, loss_seq[b] = -mean_t log(p[tgt]+1e-10),
 * dlogits = (p - onehot)/S * grad_scale ; fp32 logits [B][V][S]; dlogits may equal logits.
 * stories_cpu_ops.h:71-108 ; grad_scale is train.m:497 */
int ane_cuda_cross_entropy_dev(void *stream, ane_idtype idtype, int B, int V, int S,
                               float *dlogits, const float *logits, const void *targets,
                               float *loss_seq, float grad_scale);
/* a12 (+a13 folded): Adam over a flat fp32 range.  g is first multiplied by gscale and then by
 * *clip_dev (a device scalar, NULL = 1), as train.m:750-767 and :809-825 do in two passes.
 * flags = ANE_ADAM_STORIES or ANE_ADAM_DYNAMIC. */
int ane_cuda_adam_dev(void *stream, size_t n, float *w, const float *g, float *m, float *v, int t,
                      float lr, float b1, float b2, float eps, float wd, float gscale,
                      const float *clip_dev, unsigned flags);
/* a13: *out_dev = sum_i (g[i]*gscale)^2, fixed summation order.        train.m:770-788 */
int ane_cuda_grad_norm_sq_dev(void *stream, size_t n, const float *g, float gscale, float *out_dev);
/* a13: *factor_dev = clip/norm if clip > 0 and norm > clip else 1, norm = sqrt(sum of the
 * n_terms partial squares at normsq_dev).                               train.m:788,809-810 */
int ane_cuda_clip_factor_dev(void *stream, const float *normsq_dev, int n_terms, float clip, float *factor_dev);

/* ---- layout helpers on either side of the operators in the reference's loop --------------------------
 * GQA head tiling: x [B][kv_heads*hd][S] -> out [B][kv_heads*ratio*hd][S], every KV head repeated `ratio`
 * times (query head kv*ratio + r reads KV head kv).       training_dynamic/io.h:330-337 (gqa_tile_kv) */
int ane_cuda_gqa_tile_dev(void *stream, ane_dtype dtype, int B, int kv_heads, int ratio, int hd, int S,
                          void *out, const void *in);
/* QK-norm + RoPE of the K side written straight into the tiled (query-head) layout [B][kv_heads*ratio*hd][S]: every KV
 * head's result goes to its `ratio` query heads -- ane_cuda_qknorm_rope_dev followed by ane_cuda_gqa_tile_dev, bit for
 * bit, without the untiled tensor crossing HBM.  Head widths 64 and 128, 16-byte aligned rows (else
 * ANE_CUDA_ERR_UNSUPPORTED).                                              training_dynamic/train.m:620-621, io.h:330-337 */
int ane_cuda_qknorm_rope_tiled_dev(void *stream, ane_dtype dtype, int B, int kv_heads, int ratio, int hd, int S, void *out_tiled,
                                   const void *x, const float *w, float eps, float base, int pos0);
/* RoPE^-1 + QK-norm backward of the K side with the head sum folded in: dy_tiled is the gradient in the tiled
 * (query-head) layout [B][kv_heads*ratio*hd][S] that SDPA backward produces; the `ratio` heads of each KV head are
 * added in fp32 in head order and rounded once to the storage type, then the operator runs as
 * ane_cuda_rope_qknorm_bwd_dev -- the result equals ane_cuda_gqa_reduce_dev followed by that call bit for bit, and
 * the reduced tensor never crosses HBM.  Ratios 2 and 4 (1 forwards to the plain call), head widths 64 and 128,
 * 16-byte aligned rows; other shapes return ANE_CUDA_ERR_UNSUPPORTED.   training_dynamic/train.m:653-656, io.h:340-351 */
int ane_cuda_rope_qknorm_bwd_gqa_dev(void *stream, ane_dtype dtype, int B, int kv_heads, int ratio, int hd, int S, void *dx,
                                     float *dw, const void *dy_tiled, const void *x, const float *w, float eps, float base,
                                     int pos0, unsigned flags);
/* GQA head sum: in [B][kv_heads*ratio*hd][S] -> out [B][kv_heads*hd][S], out = 0 + in[r=0] + in[r=1] + ...
 * in head order (fp32 adds, one rounding on store).        training_dynamic/io.h:340-351 (gqa_reduce_kv) */
int ane_cuda_gqa_reduce_dev(void *stream, ane_dtype dtype, int B, int kv_heads, int ratio, int hd, int S,
                            void *out, const void *in);
/* dst[i] = (dst type) src[i], round to nearest even; any pair of f32 / f16 / bf16.
 *                                          stories_io.h:41-58, io.h:33-50 (cvt_f16_f32, cvt_f32_f16) */
int ane_cuda_convert_dev(void *stream, ane_dtype dst_dtype, ane_dtype src_dtype, size_t n, void *dst, const void *src);
/* Packed surface of the dynamic-weight matmul: row d of buf [ic][seq+oc] (16-bit) = act[d][0..seq) followed
 * by W[d][0..oc), both converted from fp32.                                   io.h:79-88 (io_write_dyn).
 * Reading a result back (io_read_dyn, io.h:91-95) is ane_cuda_convert_dev. */
int ane_cuda_pack_dyn_dev(void *stream, ane_dtype dst_dtype, int ic, int seq, int oc, void *buf,
                          const float *act, const float *W);
/* Vocabulary compaction.  full_to_compact[v] = rank of v among the ids that occur in tokens, or -1;
 * compact_to_full is its inverse (room for full_vocab entries); *compact_vocab = number of ids in use.
 * All three outputs are device memory; ids outside [0, full_vocab) are counted in the status words.
 *                                                                 cpu_ops.h:96-126 (vocab_map_build) */
int ane_cuda_vocab_map_build_dev(void *stream, ane_idtype idtype, size_t n_tokens, const void *tokens, int full_vocab,
                                 int *full_to_compact, int *compact_to_full, int *compact_vocab);
/* Rows of `dim` floats moved between the full and the compact table.  The number of rows is
 * min(*compact_vocab_dev, compact_vocab_max) when compact_vocab_dev is given (device pointer written by
 * ane_cuda_vocab_map_build_dev: no host round trip), else compact_vocab_max.
 *   compact_embed:  compact[c]          = full[compact_to_full[c]]        cpu_ops.h:129-134
 *   scatter_grads:  full[compact_to_full[c]] += compact[c]                cpu_ops.h:137-143
 *   update_full:    full[compact_to_full[c]]  = compact[c]                cpu_ops.h:146-149 */
int ane_cuda_vocab_compact_embed_dev(void *stream, float *compact_embed, const float *full_embed, const int *compact_to_full,
                                     const int *compact_vocab_dev, int compact_vocab_max, int dim, int full_vocab);
int ane_cuda_vocab_scatter_grads_dev(void *stream, float *full_gembed, const float *compact_gembed, const int *compact_to_full,
                                     const int *compact_vocab_dev, int compact_vocab_max, int dim, int full_vocab);
int ane_cuda_vocab_update_full_dev(void *stream, float *full_embed, const float *compact_embed, const int *compact_to_full,
                                   const int *compact_vocab_dev, int compact_vocab_max, int dim, int full_vocab);

/* ---- sharded optimizer step over peer memory (one process per GPU, every rank's flat gradient and parameter
 * buffers mapped into every rank: CUDA IPC or symmetric memory).  No counterpart in the reference, which is a
 * single-device program; the arithmetic is the reference's (train.m:770-869, cpu_ops.h:56-64).
 * reduce: g_slice[i] = sum over ranks r = 0..nranks-1 (in that order) of g_ranks[r][lo + i], i < n -- the
 *         reduce-scatter, read from the peers' memory -- and *normsq_dev = sum_i (g_slice[i]*gscale)^2 in a fixed
 *         order (the caller all-reduces this scalar over the ranks for the clipping norm).  scratch: NULL, or 1184
 *         floats of device memory for the block partials -- required when the call runs on a stream of its own
 *         beside other operators of this library (they share the library-owned scratch range).
 * adam:   Adam on the slice (arguments as ane_cuda_adam_dev; g_slice, m_slice, v_slice start at the slice) with the
 *         new weights stored to position lo of EVERY rank's buffer w_ranks[r] -- the all-gather.
 * g_ranks / w_ranks are host arrays of nranks (<= 8) device pointers.  The kernels never wait for another rank:
 * the caller must order "all gradients complete" before reduce, "all reduces complete" before gradients are
 * overwritten, and "all adam kernels complete" before parameters are read, across the ranks (any collective on
 * the same stream does). */
int ane_cuda_p2p_reduce_dev(void *stream, int nranks, const float *const *g_ranks, size_t lo, size_t n, float *g_slice,
                            float gscale, float *normsq_dev, float *scratch);
/* The same reduce on at most max_blocks thread blocks (0: no limit): for a reduce that runs on a side stream beside the
 * operator chain and must leave the SMs to it.  The block count is part of the (fixed) summation order of normsq. */
int ane_cuda_p2p_reduce_limited_dev(void *stream, int nranks, const float *const *g_ranks, size_t lo, size_t n, float *g_slice,
                                    float gscale, float *normsq_dev, float *scratch, int max_blocks);
int ane_cuda_p2p_adam_dev(void *stream, int nranks, int self, float *const *w_ranks, size_t lo, size_t n, const float *g_slice,
                          float *m_slice, float *v_slice, int t, float lr, float b1, float b2, float eps, float wd, float gscale,
                          const float *clip_dev, unsigned flags);

/* ---- the operator chain of one micro-batch with host buffers on the contraction side ---------------------------
 * The arrangement of the reference's loop (training_dynamic/train.m:428-482 forward, :527-720 backward): the
 * contractions run elsewhere and hand their results over in HOST memory, the operators between them run here.
 * One ane_cuda_chain_step uploads, per layer, what the contractions produced (q, k, attention output, h1, h3, FFN
 * output; dsilu, dx_ffn, dq, dk, dx_attn), runs the operators in the reference's order and downloads what the next
 * contraction consumes (xnorm, rotated q and k, x2norm, gate; dh1, dh3, dq, dk), on three streams so that copies
 * and operators of neighbouring layers overlap -- which one blocking ane_cuda_*_host call per operator cannot do.
 * The residual stream, x2 and the running gradient stay on the device; the norm-weight and embedding gradients
 * are accumulated into the caller's device buffers.  Page-locked host buffers (ane_cuda_host_alloc) are needed
 * for the overlap.  All tensors are [n_seqs][channels][seq] of `dtype`; every table below holds `layers` pointers
 * (the same pointer may be given for several layers). */
typedef struct {
    int layers, dim, hidden, heads, kv_heads, head_dim, seq, vocab;
    ane_dtype dtype;
    float alpha, eps, qk_eps, rope_base;
    unsigned norm_bwd_flags;         /* ANE_NORM_BWD_REFERENCE or ANE_NORM_BWD_EXACT */
    int rotate;                      /* device buffer sets the contraction-side tensors rotate through (>= 1; 4 is a good value) */
} ane_chain_config;
typedef struct {                     /* device pointers the caller owns */
    const float *att_w, *ffn_w;      /* [layers][dim] */
    const float *final_w;            /* [dim] */
    const float *q_w, *k_w;          /* [layers][head_dim] */
    float *att_g, *ffn_g, *final_g, *q_g, *k_g;   /* gradients of the above, accumulated into */
    const void *table;               /* [vocab][dim] of dtype */
    float *embed_g;                  /* [vocab][dim] fp32, accumulated into */
} ane_chain_params;
typedef struct {
    const void *const *q, *const *k, *const *o_out, *const *h1, *const *h3, *const *ffn_out;     /* forward, host -> device */
    void *const *xnorm, *const *q_r, *const *k_r, *const *x2norm, *const *gate;                  /* forward, device -> host */
    const void *const *dsilu, *const *dx_ffn, *const *dq_in, *const *dk_in, *const *dx_attn;     /* backward, host -> device */
    void *const *dh1, *const *dh3, *const *dq, *const *dk;                                       /* backward, device -> host */
    const void *dy_cls;              /* [n_seqs][dim][seq]: gradient entering the final norm */
    void *x_final;                   /* [n_seqs][dim][seq]: output of the final norm */
    const int32_t *tokens;           /* [n_seqs][seq] */
} ane_chain_host_io;
typedef struct ANECudaChain ANECudaChain;
ANECudaChain *ane_cuda_chain_create(const ane_chain_config *cfg, int n_seqs, const ane_chain_params *params);   /* NULL on failure */
/* Enqueues one forward + backward pass; returns before the work is done.  The host buffers must stay valid and
 * unchanged until ane_cuda_chain_sync (or the next step's completion). */
int ane_cuda_chain_step(ANECudaChain *chain, const ane_chain_host_io *io);
int ane_cuda_chain_sync(ANECudaChain *chain);
void *ane_cuda_chain_compute_stream(ANECudaChain *chain);       /* the stream the operators run on (to order an optimizer step after it) */
size_t ane_cuda_chain_h2d_bytes(const ANECudaChain *chain);     /* bytes one step copies host -> device */
size_t ane_cuda_chain_d2h_bytes(const ANECudaChain *chain);     /* and device -> host */
void ane_cuda_chain_destroy(ANECudaChain *chain);

/* ---- the multi-GPU group: one process per GPU, NCCL (loaded at run time) as the transport -----------------------
 * The reference is a single-process program; its optimizer step is the scale / norm / clip of
 * training_dynamic/train.m:750-825 followed by the per-tensor Adam loop of :837-869.  Style of these calls:
 * bridge/ane_bridge.h:20-68 (int status, explicit create / destroy).
 *   unique_id  rank 0 makes the 128-byte id and hands it to the other ranks by any means (a file, MPI, a socket).
 *   init       joins the group on the CURRENT device (after ane_cuda_init).  timeout_s bounds this call and becomes the
 *              default for the waits below; a rank that never joins ends it with ANE_CUDA_ERR_TIMEOUT, and the
 *              half-made communicator is aborted.
 *   allreduce  sum over the ranks, in place, on the stream (the scalar loss of a data-parallel step).
 *   wait       host-side wait for the stream with a deadline (timeout_s < 0: the default): polls the stream and the
 *              communicator; on a timeout or a communicator error the communicator is ABORTED (so that a collective
 *              kernel waiting for a missing rank ends) and an error code is returned.  The group must then be rebuilt.
 *   map_peers  optional, collective, blocking: exchanges CUDA IPC handles of the flat parameter and gradient buffers
 *              so that the sharded step below runs on this library's peer-memory kernels instead of NCCL's
 *              reduce-scatter / all-gather.  ANE_CUDA_ERR_UNSUPPORTED where the ranks cannot map each other.
 *   sharded_adam_step   the whole optimizer step over flat fp32 buffers of n_padded floats (a multiple of the rank
 *              count): reduce-scatter of g, squared norm of (g * gscale), one clip factor for all ranks
 *              (clip <= 0: none), Adam on this rank's slice with weight decay on [0, n_decay) and none on
 *              [n_decay, n_params), all-gather of w.  Asynchronous on the stream; normsq_out (device, may be NULL)
 *              receives the squared norm.  Every rank must call it with the same arguments.  With one rank it is
 *              the plain local step. */
#define ANE_CUDA_COMM_ID_BYTES 128
#define ANE_CUDA_MAX_RANKS 8
int ane_cuda_comm_unique_id(void *id_out);
int ane_cuda_comm_init(int nranks, int rank, const void *id, double timeout_s);
int ane_cuda_comm_size(void);
int ane_cuda_comm_rank(void);
int ane_cuda_comm_destroy(void);
int ane_cuda_comm_wait(void *stream, double timeout_s);
int ane_cuda_allreduce_f32(void *stream, float *buf, size_t n);
int ane_cuda_comm_map_peers(float *w, float *g, size_t n_floats);
int ane_cuda_comm_unmap_peers(void);
int ane_cuda_sharded_adam_step(void *stream, float *w, float *g, float *m, float *v, size_t n_padded, size_t n_decay,
                               size_t n_params, int t, float lr, float b1, float b2, float eps, float wd, float gscale,
                               float clip, unsigned flags, float *normsq_out);

/* ---- checkpoints of the reference's training loops ("BLZT" files) ------------------------------------
 * Header as written by save_checkpoint: version 2 (training/stories_config.h:95-104, train_large.m:109-145;
 * the last three ints are padding) and version 4 (training_dynamic/config.h:78-86, train.m:104-138). */
typedef struct {
    int magic;                 /* 0x424C5A54 */
    int version;               /* 2 or 4 */
    int step, total_steps;
    int n_layers, vocab_size, dim, hidden_dim, n_heads, seq_len;
    float lr, loss;
    double cum_compile, cum_train, cum_wall;
    int cum_steps, cum_batches, adam_t;
    int kv_heads, head_dim, q_dim;   /* version 4; padding in version 2 */
} ane_ckpt_header;
/* Reads and validates the header only (no GPU needed). */
int ane_cuda_ckpt_read_header(const char *path, ane_ckpt_header *hdr);
/* Number of parameters the file holds = floats in each of the w / m / v buffers below. 0 for a bad header. */
size_t ane_cuda_ckpt_param_count(const ane_ckpt_header *hdr);
/* File -> device.  The three device buffers receive the weights and the two Adam moments in "weight order":
 * per layer Wq Wk Wv Wo W1 W2 W3 rms_att rms_ffn, then rms_final, then embed -- the file's order with the
 * moments taken out (load_checkpoint, train.m:140-172).  m_dev and v_dev may both be NULL (weights only). */
int ane_cuda_ckpt_load(const char *path, ane_ckpt_header *hdr, float *w_dev, float *m_dev, float *v_dev, size_t n_floats);
/* Device -> file, byte-identical to what the reference's save_checkpoint writes for the same values. */
int ane_cuda_ckpt_save(const char *path, const ane_ckpt_header *hdr, const float *w_dev, const float *m_dev,
                       const float *v_dev, size_t n_floats);
/* The same files to and from "optimizer order", the arrangement a flat optimizer wants: everything that takes weight
 * decay first, the norm weights (no decay, train.m:837-869) after it --
 *   [layer 0: Wq Wk Wv Wo W1 W2 W3] ... [layer L-1: ...] embed | rms_att[all layers] rms_ffn[all layers] rms_final | extras
 * so that Adam is two range updates: [0, ane_cuda_ckpt_flat_decay_count) with decay, the rest without.  n_floats may
 * exceed the file's parameter count: floats past it (for example per-head QK-norm weights, which the reference's
 * files do not hold) are not touched by a load and not written by a save -- after loading a file into a model that
 * has them, initialise them yourself (1 for weights, 0 for moments); saving drops them. */
int ane_cuda_ckpt_load_flat(const char *path, ane_ckpt_header *hdr, float *w_dev, float *m_dev, float *v_dev, size_t n_floats);
int ane_cuda_ckpt_save_flat(const char *path, const ane_ckpt_header *hdr, const float *w_dev, const float *m_dev,
                            const float *v_dev, size_t n_floats);
size_t ane_cuda_ckpt_flat_decay_count(const ane_ckpt_header *hdr);
/* Where one tensor lies in either arrangement (flat = 0: weight order, 1: optimizer order).  tensor: 0..6 = Wq Wk Wv Wo
 * W1 W2 W3, 7 = rms_att, 8 = rms_ffn (each per layer), 9 = rms_final, 10 = embed.  No GPU needed. */
enum { ANE_T_WQ = 0, ANE_T_WK, ANE_T_WV, ANE_T_WO, ANE_T_W1, ANE_T_W2, ANE_T_W3, ANE_T_RMS_ATT, ANE_T_RMS_FFN, ANE_T_RMS_FINAL, ANE_T_EMBED };
int ane_cuda_ckpt_tensor_offset(const ane_ckpt_header *hdr, int flat, int tensor, int layer, size_t *offset, size_t *count);

/* ---- llama2.c weight files: the pretrained-weights loader of training/train_large.m:13-56 (load_pretrained).
 * Header of seven ints (stories_config.h:108-110), then embed, rms_att[all layers], wq[all], wk[all], wv[all], wo[all],
 * rms_ffn[all], w1[all], w2[all], w3[all], rms_final; a negative vocab_size marks an unshared classifier, which -- like
 * the reference -- this loader does not read.  Wk and Wv are dim * (dim * n_kv_heads / n_heads) each (equal to the
 * reference's dim * dim when n_kv_heads == n_heads, the only case it handles). */
typedef struct {
    int dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len;
} ane_llama2c_config;
/* Reads and validates the 28-byte header only (no GPU needed). */
int ane_cuda_llama2c_read_config(const char *path, ane_llama2c_config *cfg);
/* The checkpoint header describing the same model (version 2 for square attention, 4 for grouped-query; step counters
 * zero), i.e. what ane_cuda_ckpt_save needs to write these weights as a reference checkpoint. */
int ane_cuda_llama2c_to_header(const ane_llama2c_config *cfg, ane_ckpt_header *hdr);
/* File -> device weights in weight order (flat = 0) or optimizer order (flat = 1); *hdr receives the header above.
 * expect may be NULL; otherwise dim, hidden_dim and n_layers must equal the file's ("Config mismatch",
 * train_large.m:20-23).  A file shorter than its header promises is refused (ANE_CUDA_ERR_INVALID). */
int ane_cuda_llama2c_load(const char *path, const ane_llama2c_config *expect, ane_ckpt_header *hdr, float *w_dev,
                          size_t n_floats, int flat);

#ifdef __cplusplus
}
#endif
#endif /* ANE_CUDA_H */
