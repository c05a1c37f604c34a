/* oracle_ops.c -- CPU restatement of the maderix/ANE per-layer non-matmul operator set.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: only the
 * test-suite, the smoke entry and the benchmark's CPU-baseline leg may load it.  The
 * shipped library never calls into it and has no CPU fallback.
 *
 * Every function is a plain-C, fp32, single-thread restatement of the reference algorithm
 * and cites the reference lines it follows (paths relative to the reference project).
 * Tensors are channel-first: element (c, t) of one sequence lives at c*S + t
 * (training/stories_cpu_ops.h:10,117).  Functions that take `B` loop over B independent
 * sequences laid out back to back as [B][C][S].
 *
 * Parity pins: oracle rmsnorm / rmsnorm_bwd / cross-entropy / Adam / embed / RoPE-bwd are
 * checked against the reference's own functions compiled from source (oracle/_ref) and
 * against the seeded fixtures of training/test_rmsnorm_bwd.m:26-33 and
 * training/test_classifier.m:25-27,132-134 (tests/golden).  SwiGLU fwd/bwd, RoPE fwd, the
 * residual and the gradient scale / norm / clip are statements inside the reference's
 * Objective-C main file or functions of a header that includes Objective-C: they are checked
 * against those very lines, extracted by line range and compiled behind the Accelerate
 * stand-in (ref_inline_exports.c.in -> oracle/_ref/libref_inline.so), live and through golden
 * vectors.  "Parity unpinned" remains for the per-head QK-norm (the reference has none: it is
 * rmsnorm over the channels of one head, checked against the pinned rmsnorm head by head) and
 * for the GQA / cast / pack helpers (their reference header is Objective-C over IOSurface).
 */
#include <math.h>
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ RMSNorm forward
 * training/stories_cpu_ops.h:6-21 (same math as training_dynamic/cpu_ops.h:7-22):
 *   ss[t]   = sum_c x[c,t]^2                      (:9-12, accumulated channel by channel)
 *   ss[t]   = ss[t]*(1/d) + eps ; rrms = 1/sqrt   (:13-15, eps is the literal 1e-5 there)
 *   out     = (x * rrms) * w[c]                   (:16-19, in that order)               */
/* `n` tokens starting at x, channel rows `stride` floats apart (stride == n for a whole sequence). */
static void rmsnorm_s(float *out, const float *x, const float *w, int d, int n, size_t stride, float eps) {
    float *ss = (float *)calloc((size_t)n, sizeof(float));
    for (int i = 0; i < d; i++)
        for (int t = 0; t < n; t++) { float v = x[(size_t)i * stride + t]; ss[t] += v * v; }
    const float invd = 1.0f / d;
    for (int t = 0; t < n; t++) ss[t] = 1.0f / sqrtf(ss[t] * invd + eps);
    for (int i = 0; i < d; i++)
        for (int t = 0; t < n; t++) {
            float v = x[(size_t)i * stride + t] * ss[t];
            out[(size_t)i * stride + t] = v * w[i];
        }
    free(ss);
}
ORC_API void orc_rmsnorm(float *out, const float *x, const float *w, int d, int S, float eps) {
    rmsnorm_s(out, x, w, d, S, (size_t)S, eps);
}

/* Work splitting for the timed CPU baseline only: with g_chunk > 0 the batched functions cut
 * every sequence into blocks of g_chunk tokens and spread (sequence, block) pairs over the
 * OpenMP threads.  Per-token results are unchanged; token-summed results (dw) then add block
 * sums instead of one running sum, so parity runs keep g_chunk = 0 (the reference's order). */
static int g_chunk = 0;
ORC_API void orc_set_chunk(int tokens) { g_chunk = tokens > 0 ? tokens : 0; }
static int n_blocks(int S) { return g_chunk > 0 ? (S + g_chunk - 1) / g_chunk : 1; }
static void block_span(int S, int k, int *t0, int *n) {
    if (g_chunk <= 0) { *t0 = 0; *n = S; return; }
    *t0 = k * g_chunk;
    *n = S - *t0 < g_chunk ? S - *t0 : g_chunk;
}

ORC_API void orc_rmsnorm_batched(float *out, const float *x, const float *w, int B, int d, int S, float eps) {
    const int nb = n_blocks(S);
    #pragma omp parallel for schedule(static)
    for (int it = 0; it < B * nb; it++) {
        int b = it / nb, t0, n;
        block_span(S, it % nb, &t0, &n);
        rmsnorm_s(out + (size_t)b * d * S + t0, x + (size_t)b * d * S + t0, w, d, n, (size_t)S, eps);
    }
}

/* ------------------------------------------------------------------ RMSNorm backward
 * training/stories_cpu_ops.h:23-53 (= training_dynamic/cpu_ops.h:24-54):
 *   rrms[t] as in the forward                                     (:26-33)
 *   dot[t]  = sum_c (dy*x)*w[c]                                   (:35-38)
 *   dot[t] *= rrms^2 * (1/d)                                      (:39-41)
 *   dx      = ((dy - x*dot) * rrms) * w[c]      OVERWRITES dx      (:43-46)
 *   dw[c]  += sum_t (dy*x)*rrms                 ACCUMULATES        (:47-50)
 * The reference multiplies BOTH terms of dx by w[c]; this differs from the analytic
 * gradient rrms*(w*dy - x*dot) when w != 1.  `exact` != 0 selects the analytic form, which
 * is what the MIL graph in training/ane_rmsnorm_bwd.h:56,70-74 computes.                 */
static void rmsnorm_bwd_s(float *dx, float *dw, const float *dy, const float *x, const float *w,
                          int d, int S, size_t stride, float eps, int exact) {
    float *ss = (float *)calloc((size_t)S, sizeof(float));
    float *rrms = (float *)malloc((size_t)S * sizeof(float));
    float *dot = (float *)calloc((size_t)S, sizeof(float));
    for (int i = 0; i < d; i++)
        for (int t = 0; t < S; t++) { float v = x[(size_t)i * stride + t]; ss[t] += v * v; }
    const float invd = 1.0f / d;
    for (int t = 0; t < S; t++) rrms[t] = 1.0f / sqrtf(ss[t] * invd + eps);
    for (int i = 0; i < d; i++)
        for (int t = 0; t < S; t++) {
            float p = dy[(size_t)i * stride + t] * x[(size_t)i * stride + t];
            dot[t] = p * w[i] + dot[t];
        }
    for (int t = 0; t < S; t++) { float r2 = rrms[t] * rrms[t]; r2 = r2 * invd; dot[t] = dot[t] * r2; }
    for (int i = 0; i < d; i++) {
        float s = 0.0f;
        for (int t = 0; t < S; t++) {
            size_t k = (size_t)i * stride + t;
            if (exact) {
                float a = dy[k] * w[i];
                float b = x[k] * dot[t];
                dx[k] = (a - b) * rrms[t];
            } else {
                float tmp = x[k] * dot[t];
                tmp = dy[k] - tmp;
                tmp = tmp * rrms[t];
                dx[k] = tmp * w[i];
            }
            float q = dy[k] * x[k];
            s += q * rrms[t];
        }
        dw[i] += s;
    }
    free(ss); free(rrms); free(dot);
}
ORC_API void orc_rmsnorm_bwd(float *dx, float *dw, const float *dy, const float *x, const float *w,
                             int d, int S, float eps, int exact) {
    rmsnorm_bwd_s(dx, dw, dy, x, w, d, S, (size_t)S, eps, exact);
}

/* Batched form.  dw accumulates over the B sequences in order b = 0..B-1, as the reference's
 * accumulation steps would (training_dynamic/train.m:588,719 called once per step). */
ORC_API void orc_rmsnorm_bwd_batched(float *dx, float *dw, const float *dy, const float *x, const float *w,
                                     int B, int d, int S, float eps, int exact) {
    /* per-sequence dw rows, then added in order b = 0..B-1: the same additions as accumulating
     * into dw call after call, but the sequences can run on separate threads */
    const int nb = n_blocks(S);
    float *dwl = (float *)calloc((size_t)B * nb * d, sizeof(float));
    #pragma omp parallel for schedule(static)
    for (int it = 0; it < B * nb; it++) {
        int b = it / nb, t0, n;
        block_span(S, it % nb, &t0, &n);
        size_t o = (size_t)b * d * S + t0;
        rmsnorm_bwd_s(dx + o, dwl + (size_t)it * d, dy + o, x + o, w, d, n, (size_t)S, eps, exact);
    }
    for (int it = 0; it < B * nb; it++)
        for (int i = 0; i < d; i++) dw[i] += dwl[(size_t)it * d + i];
    free(dwl);
}

/* ------------------------------------------------------------------ DeepNet-alpha residual
 * training/training_dynamic/train.m:460  x2 = o_out*alpha + x  (vDSP_vsma)
 * training/training_dynamic/mil_dynamic.h:279-283  x_next = x2 + alpha*ffn_out
 * training/train_large.m:427,442 is the alpha = 1 case.                                  */
ORC_API void orc_residual(float *out, const float *x, const float *f, float alpha, size_t n) {
    #pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) out[i] = f[i] * alpha + x[i];
}
/* train.m:523,595  y = alpha * x ;  train.m:497 dlogits *= loss_scale */
ORC_API void orc_scale(float *out, const float *x, float alpha, size_t n) {
    #pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) out[i] = x[i] * alpha;
}
/* train.m:590,714,721  out = a + b */
ORC_API void orc_add(float *out, const float *a, const float *b, size_t n) {
    #pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) out[i] = a[i] + b[i];
}

/* ------------------------------------------------------------------ SiLU / SwiGLU gate forward
 * training/forward.h:101  silu_f(x) = x / (1 + expf(-x));  :149-151  out = silu_f(h1) * h3
 * (the ANE graphs compute h1*sigmoid(h1)*h3: stories_mil.h:99-101, mil_dynamic.h:264-266) */
ORC_API void orc_swiglu(float *out, const float *h1, const float *h3, size_t n) {
    #pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        float s = h1[i] / (1.0f + expf(-h1[i]));
        out[i] = s * h3[i];
    }
}

/* ------------------------------------------------------------------ SwiGLU backward
 * training/training_dynamic/train.m:537-554, pass by pass:
 *   sig  = 1 / (1 + exp(-h1))
 *   dh3  = dsilu * (h1 * sig)
 *   t2   = sig * (1 + h1 * (-(sig - 1)))
 *   dh1  = (dsilu * h3) * t2                                                            */
ORC_API void orc_swiglu_bwd(float *dh1, float *dh3, const float *h1, const float *h3,
                            const float *dsilu, size_t n) {
    #pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        float e = expf(h1[i] * -1.0f);
        float sig = 1.0f / (e + 1.0f);
        float a = h1[i] * sig;
        dh3[i] = dsilu[i] * a;
        float t2 = sig + -1.0f;
        t2 = -t2;
        t2 = h1[i] * t2;
        t2 = t2 + 1.0f;
        t2 = sig * t2;
        float b = dsilu[i] * h3[i];
        dh1[i] = b * t2;
    }
}

/* ------------------------------------------------------------------ RoPE forward / backward
 * Channel-first indexing and the backward rotation: training_dynamic/cpu_ops.h:168-184.
 * Forward rotation: training/forward.h:55-70 and mil_dynamic.h:145-153 (interleaved pairs
 * (2i, 2i+1) inside a head; (a,b) -> (a cos - b sin, a sin + b cos)).
 *   freq  = 1 / powf(base, 2*i/hd)   (cpu_ops.h:172, base is the literal 10000 there)
 *   theta = p * freq ; p counted from pos0 (0 in the reference)
 * inverse != 0 gives the backward (transposed) rotation (a cos + b sin, -a sin + b cos). */
static void rope_s(float *x, int seq, size_t stride, int dim, int hd, float base, int pos0, int inverse) {
    int nheads = dim / hd;
    for (int h = 0; h < nheads; h++)
        for (int i = 0; i < hd / 2; i++) {
            float freq = 1.0f / powf(base, 2.0f * i / (float)hd);
            for (int p = 0; p < seq; p++) {
                float theta = (p + pos0) * freq;
                float c = cosf(theta), s = sinf(theta);
                size_t i0 = (size_t)(h * hd + 2 * i) * stride + p;
                size_t i1 = (size_t)(h * hd + 2 * i + 1) * stride + p;
                float v0 = x[i0], v1 = x[i1];
                if (inverse) { x[i0] = v0 * c + v1 * s;  x[i1] = -v0 * s + v1 * c; }
                else         { x[i0] = v0 * c - v1 * s;  x[i1] = v0 * s + v1 * c; }
            }
        }
}
ORC_API void orc_rope(float *x, int seq, int dim, int hd, float base, int pos0, int inverse) {
    rope_s(x, seq, (size_t)seq, dim, hd, base, pos0, inverse);
}
ORC_API void orc_rope_batched(float *x, int B, int seq, int dim, int hd, float base, int pos0, int inverse) {
    const int nb = n_blocks(seq);
    #pragma omp parallel for schedule(static)
    for (int it = 0; it < B * nb; it++) {
        int b = it / nb, t0, n;
        block_span(seq, it % nb, &t0, &n);
        rope_s(x + (size_t)b * dim * seq + t0, n, (size_t)seq, dim, hd, base, pos0 + t0, inverse);
    }
}

/* ------------------------------------------------------------------ per-head QK-RMSNorm
 * Not in the reference.  Defined as the RMSNorm of stories_cpu_ops.h:6-53 with the reduction
 * taken over the hd channels of one head, one weight vector w[hd] shared by all heads. */
ORC_API void orc_qknorm(float *out, const float *x, const float *w, int heads, int hd, int S, float eps) {
    for (int h = 0; h < heads; h++)
        orc_rmsnorm(out + (size_t)h * hd * S, x + (size_t)h * hd * S, w, hd, S, eps);
}
ORC_API void orc_qknorm_bwd(float *dx, float *dw, const float *dy, const float *x, const float *w,
                            int heads, int hd, int S, float eps, int exact) {
    for (int h = 0; h < heads; h++)
        orc_rmsnorm_bwd(dx + (size_t)h * hd * S, dw, dy + (size_t)h * hd * S, x + (size_t)h * hd * S,
                        w, hd, S, eps, exact);
}
/* Fused forward: out = rope(qknorm(x)); fused backward: dx = qknorm_bwd(rope^-1(dy), x). */
ORC_API void orc_qknorm_rope_batched(float *out, const float *x, const float *w, int B, int heads, int hd,
                                     int S, float eps, float base, int pos0) {
    const int nb = n_blocks(S);
    #pragma omp parallel for schedule(static)
    for (int it = 0; it < B * nb; it++) {
        int b = it / nb, t0, n;
        block_span(S, it % nb, &t0, &n);
        size_t o = (size_t)b * heads * hd * S + t0;
        for (int h = 0; h < heads; h++)
            rmsnorm_s(out + o + (size_t)h * hd * S, x + o + (size_t)h * hd * S, w, hd, n, (size_t)S, eps);
        rope_s(out + o, n, (size_t)S, heads * hd, hd, base, pos0 + t0, 0);
    }
}
ORC_API void orc_rope_qknorm_bwd_batched(float *dx, float *dw, const float *dy, const float *x, const float *w,
                                         int B, int heads, int hd, int S, float eps, float base, int pos0,
                                         int exact) {
    const size_t n = (size_t)heads * hd * S;
    const int nb = n_blocks(S);
    float *dwl = (float *)calloc((size_t)B * nb * heads * hd, sizeof(float));
    #pragma omp parallel for schedule(static)
    for (int it = 0; it < B * nb; it++) {
        int b = it / nb, t0, m;
        block_span(S, it % nb, &t0, &m);
        /* g = rope^-1(dy) for this block, packed with row stride m */
        float *g = (float *)malloc((size_t)heads * hd * m * sizeof(float));
        for (int c = 0; c < heads * hd; c++)
            memcpy(g + (size_t)c * m, dy + (size_t)b * n + (size_t)c * S + t0, (size_t)m * sizeof(float));
        rope_s(g, m, (size_t)m, heads * hd, hd, base, pos0 + t0, 1);
        /* the norm backward reads g with stride m and x / dx with stride S: go head by head through a
         * strided copy of x so one routine serves both */
        float *xb = (float *)malloc((size_t)hd * m * sizeof(float));
        float *db = (float *)malloc((size_t)hd * m * sizeof(float));
        for (int h = 0; h < heads; h++) {   /* one dw row per (sequence, block, head), summed in order below */
            const size_t o = (size_t)b * n + (size_t)h * hd * S + t0;
            for (int c = 0; c < hd; c++) memcpy(xb + (size_t)c * m, x + o + (size_t)c * S, (size_t)m * sizeof(float));
            rmsnorm_bwd_s(db, dwl + ((size_t)it * heads + h) * hd, g + (size_t)h * hd * m, xb, w, hd, m, (size_t)m, eps, exact);
            for (int c = 0; c < hd; c++) memcpy(dx + o + (size_t)c * S, db + (size_t)c * m, (size_t)m * sizeof(float));
        }
        free(g); free(xb); free(db);
    }
    for (size_t r = 0; r < (size_t)B * nb * heads; r++)
        for (int i = 0; i < hd; i++) dw[i] += dwl[r * hd + i];
    free(dwl);
}

/* ------------------------------------------------------------------ embedding gather / scatter-add
 * training/stories_cpu_ops.h:112-131 (training_dynamic/cpu_ops.h:150-164 is the same without
 * the range check).  An out-of-range id leaves the column of x untouched and is skipped by the
 * backward pass (stories_cpu_ops.h:115,126).  Returns the number of out-of-range ids.      */
ORC_API int orc_embed_lookup(float *x, const float *embed, const int32_t *tokens, int dim, int seq, int vocab) {
    int oor = 0;
    for (int t = 0; t < seq; t++) {
        int tok = tokens[t];
        if (tok < 0 || tok >= vocab) { oor++; continue; }
        for (int d = 0; d < dim; d++) x[(size_t)d * seq + t] = embed[(size_t)tok * dim + d];
    }
    return oor;
}
ORC_API int orc_embed_backward(float *d_embed, const float *dx, const int32_t *tokens, int dim, int seq, int vocab) {
    int oor = 0;
    for (int t = 0; t < seq; t++) {
        int tok = tokens[t];
        if (tok < 0 || tok >= vocab) { oor++; continue; }
        for (int d = 0; d < dim; d++) d_embed[(size_t)tok * dim + d] += dx[(size_t)d * seq + t];
    }
    return oor;
}

/* ------------------------------------------------------------------ softmax cross-entropy fwd+bwd
 * training/stories_cpu_ops.h:71-108 and training_dynamic/cpu_ops.h:68-93, per token t:
 *   m = max_v l ; e = exp(l - m) ; p = e * (1/sum e)
 *   loss -= logf(p[tgt] + 1e-10)      (epsilon inside the log)
 *   p[tgt] -= 1 ; dlogits = p * (1/S) ; returns loss / S
 * Out-of-range target (stories variant, :94-103): the column keeps the plain softmax (no -1,
 * no 1/S) and adds nothing to the loss, while the loss still divides by S.
 * grad_scale multiplies dlogits afterwards (training_dynamic/train.m:497, loss_scale).
 * Returns the loss; *n_oor (may be NULL) receives the count of out-of-range targets.      */
ORC_API float orc_cross_entropy(float *dlogits, const float *logits, const int32_t *targets, int V, int S,
                                float grad_scale, int *n_oor) {
    float total = 0.0f;
    const float invS = 1.0f / S;
    int oor = 0;
    float *col = (float *)malloc((size_t)V * sizeof(float));
    for (int t = 0; t < S; t++) {
        float m = -INFINITY;
        for (int v = 0; v < V; v++) { float l = logits[(size_t)v * S + t]; if (l > m) m = l; }
        float sum = 0.0f;
        const float negm = -m;
        for (int v = 0; v < V; v++) { col[v] = expf(logits[(size_t)v * S + t] + negm); sum += col[v]; }
        const float inv = 1.0f / sum;
        for (int v = 0; v < V; v++) col[v] = col[v] * inv;
        int tgt = targets[t];
        if (tgt < 0 || tgt >= V) {
            oor++;
        } else {
            total -= logf(col[tgt] + 1e-10f);
            col[tgt] -= 1.0f;
            for (int v = 0; v < V; v++) col[v] = col[v] * invS;
        }
        if (grad_scale != 1.0f) for (int v = 0; v < V; v++) col[v] = col[v] * grad_scale;
        for (int v = 0; v < V; v++) dlogits[(size_t)v * S + t] = col[v];
    }
    free(col);
    if (n_oor) *n_oor = oor;
    return total / S;
}

/* ------------------------------------------------------------------ Adam
 * variant 0: training/stories_cpu_ops.h:55-63     w -= lr * mh / (sqrtf(vh) + eps)
 * variant 1: training_dynamic/cpu_ops.h:56-64     w -= lr * (mh / (sqrtf(vh) + eps) + wd * w)
 * Bias corrections use powf(b, t) with the int step converted to float (:56 / :57).
 * gscale and clip multiply the gradient first, in two separate roundings, as
 * training_dynamic/train.m:750-767 (scale) and :809-825 (clip) do before calling Adam.   */
ORC_API void orc_adam(float *w, const float *g, float *m, float *v, size_t n, int t, float lr,
                      float b1, float b2, float eps, float wd, int variant, float gscale, float clip) {
    float bc1 = 1.0f - powf(b1, t), bc2 = 1.0f - powf(b2, t);
    #pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        float gi = g[i];
        if (gscale != 1.0f) gi = gi * gscale;
        if (clip != 1.0f) gi = gi * clip;
        m[i] = b1 * m[i] + (1 - b1) * gi;
        v[i] = b2 * v[i] + (1 - b2) * gi * gi;
        float mh = m[i] / bc1, vh = v[i] / bc2;
        if (variant == 0) w[i] -= lr * mh / (sqrtf(vh) + eps);
        else              w[i] -= lr * (mh / (sqrtf(vh) + eps) + wd * w[i]);
    }
}

/* ------------------------------------------------------------------ gradient post-processing
 * training_dynamic/train.m:750-767  g *= gsc ; :770-788  norm^2 = sum over tensors of
 * dot(g,g) (fp32 running sums) ; :809-825  if norm > clip: g *= clip/norm.
 * orc_grad_norm_sq returns sum (g*gscale)^2 in double so that it can arbitrate between two
 * fp32 summation orders; orc_clip_factor restates the branch at :809-810.                 */
ORC_API double orc_grad_norm_sq(const float *g, size_t n, float gscale) {
    double s = 0.0;
    for (size_t i = 0; i < n; i++) { float gi = g[i] * gscale; s += (double)gi * (double)gi; }
    return s;
}
ORC_API float orc_clip_factor(float norm_sq, float clip) {
    float norm = sqrtf(norm_sq);
    if (clip > 0.0f && norm > clip) return clip / norm;
    return 1.0f;
}

/* ------------------------------------------------------------------ vocab compaction
 * training_dynamic/cpu_ops.h:102-125: mark ids that occur, number them in increasing id
 * order; returns the compact vocabulary size.                                            */
ORC_API int orc_vocab_map_build(const int32_t *data, size_t n_tokens, int full_vocab,
                                int32_t *full_to_compact, int32_t *compact_to_full) {
    for (int v = 0; v < full_vocab; v++) full_to_compact[v] = -1;
    for (size_t i = 0; i < n_tokens; i++) full_to_compact[data[i]] = 0;
    int cid = 0;
    for (int v = 0; v < full_vocab; v++) {
        if (full_to_compact[v] == 0) { full_to_compact[v] = cid; compact_to_full[cid] = v; cid++; }
        else full_to_compact[v] = -1;
    }
    return cid;
}

/* training_dynamic/cpu_ops.h:129-134: compact table = rows of the full table in compact order */
ORC_API void orc_vocab_compact_embed(float *compact, const float *full_embed, const int32_t *compact_to_full, int compact_vocab, int dim) {
    for (int c = 0; c < compact_vocab; c++)
        memcpy(compact + (size_t)c * dim, full_embed + (size_t)compact_to_full[c] * dim, (size_t)dim * 4);
}
/* cpu_ops.h:137-143: full gradient rows += compact gradient rows */
ORC_API void orc_vocab_scatter_grads(float *full_gembed, const float *compact_gembed, const int32_t *compact_to_full, int compact_vocab, int dim) {
    for (int c = 0; c < compact_vocab; c++) {
        const int fv = compact_to_full[c];
        for (int d = 0; d < dim; d++) full_gembed[(size_t)fv * dim + d] += compact_gembed[(size_t)c * dim + d];
    }
}
/* cpu_ops.h:146-149: full table rows = compact rows (after the optimizer step) */
ORC_API void orc_vocab_update_full(float *full_embed, const float *compact_embed, const int32_t *compact_to_full, int compact_vocab, int dim) {
    for (int c = 0; c < compact_vocab; c++)
        memcpy(full_embed + (size_t)compact_to_full[c] * dim, compact_embed + (size_t)c * dim, (size_t)dim * 4);
}

/* ------------------------------------------------------------------ GQA helpers
 * training_dynamic/io.h:330-337: every KV head copied to its `ratio` query heads. in [kv_heads*hd, seq] */
ORC_API void orc_gqa_tile_kv(float *out, const float *in, int kv_heads, int ratio, int hd, int seq) {
    for (int kv = 0; kv < kv_heads; kv++)
        for (int r = 0; r < ratio; r++)
            memcpy(out + (size_t)(kv * ratio + r) * hd * seq, in + (size_t)kv * hd * seq, (size_t)hd * seq * sizeof(float));
}
/* io.h:340-351: zero, then add the query heads of each KV head in head order */
ORC_API void orc_gqa_reduce_kv(float *out, const float *in, int kv_heads, int ratio, int hd, int seq) {
    memset(out, 0, (size_t)kv_heads * hd * seq * sizeof(float));
    for (int kv = 0; kv < kv_heads; kv++)
        for (int r = 0; r < ratio; r++) {
            const float *src = in + (size_t)(kv * ratio + r) * hd * seq;
            float *dst = out + (size_t)kv * hd * seq;
            for (size_t i = 0; i < (size_t)hd * seq; i++) dst[i] += src[i];
        }
}

/* ------------------------------------------------------------------ fp32 <-> fp16 and the packed surface
 * stories_io.h:41-58 / io.h:33-50: element-wise casts (NEON vcvt = round to nearest even, as the C cast). */
ORC_API void orc_cvt_f32_f16(uint16_t *dst, const float *src, size_t n) {
    for (size_t i = 0; i < n; i++) { const _Float16 h = (_Float16)src[i]; memcpy(dst + i, &h, 2); }
}
ORC_API void orc_cvt_f16_f32(float *dst, const uint16_t *src, size_t n) {
    for (size_t i = 0; i < n; i++) { _Float16 h; memcpy(&h, src + i, 2); dst[i] = (float)h; }
}
/* io.h:79-88 (io_write_dyn): row d = act[d][0..seq) then W[d][0..oc), fp16 */
ORC_API void orc_pack_dyn_f16(uint16_t *buf, const float *act, int ic, int seq, const float *W, int oc) {
    const int sp = seq + oc;
    for (int d = 0; d < ic; d++) {
        orc_cvt_f32_f16(buf + (size_t)d * sp, act + (size_t)d * seq, (size_t)seq);
        orc_cvt_f32_f16(buf + (size_t)d * sp + seq, W + (size_t)d * oc, (size_t)oc);
    }
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
