/* A C caller of libane_cuda in the order of the reference's training step (training/train_large.m:395-660,
 * training_dynamic/train.m:405-870): host float arrays from malloc, the reference's own function signatures,
 * one sequence.  The contractions of the real loop (QKV / output / FFN projections, SDPA, classifier) are
 * replaced by pseudo-random fills, as they are not part of this library.  Every operator result is compared
 * with the CPU oracle (liboracle: a C restatement of the reference's functions); exit code 0 when all agree
 * to 1e-5 of the tensor's largest magnitude, else the number of mismatching operators.
 *
 * Build: gcc train_step_driver.c -I<include> -L<libdir> -lane_cuda -L<oracledir> -loracle -lm */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "ane_cuda.h"

/* oracle (test infrastructure) */
void orc_rmsnorm(float *out, const float *x, const float *w, int d, int S, float eps);
void orc_rmsnorm_bwd(float *dx, float *dw, const float *dy, const float *x, const float *w, int d, int S, float eps, int exact);
void orc_residual(float *out, const float *x, const float *f, float alpha, size_t n);
void orc_swiglu(float *out, const float *h1, const float *h3, size_t n);
void orc_swiglu_bwd(float *dh1, float *dh3, const float *h1, const float *h3, const float *d, size_t n);
void orc_rope(float *x, int seq, int dim, int hd, float base, int pos0, int inverse);
int orc_embed_lookup(float *x, const float *embed, const int32_t *tokens, int dim, int seq, int vocab);
int orc_embed_backward(float *d_embed, const float *dx, const int32_t *tokens, int dim, int seq, int vocab);
float orc_cross_entropy(float *dlogits, const float *logits, const int32_t *targets, int V, int S, float grad_scale, int *n_oor);
void orc_adam(float *w, const float *g, float *m, float *v, size_t n, int t, float lr, float b1, float b2, float eps, float wd,
              int variant, float gscale, float clip);

enum { DIM = 768, SEQ = 256, HIDDEN = 2048, VOCAB = 4096, HD = 64 };

static uint64_t g_state = 0x9E3779B97F4A7C15ull;
static float frand(void) {          /* xorshift, roughly N(0,1) by summing uniforms */
    float s = 0.0f;
    for (int i = 0; i < 4; i++) {
        g_state ^= g_state << 13; g_state ^= g_state >> 7; g_state ^= g_state << 17;
        s += (float)(g_state >> 40) / 16777216.0f;
    }
    return (s - 2.0f) * 1.7320508f;
}
static float *filled(size_t n, float scale) {
    float *p = (float *)malloc(n * sizeof(float));
    for (size_t i = 0; i < n; i++) p[i] = scale * frand();
    return p;
}
static float *zeros(size_t n) { return (float *)calloc(n, sizeof(float)); }

static int g_bad = 0;
static void check(const char *what, const float *got, const float *want, size_t n) {
    double worst = 0.0, scale = 0.0;
    for (size_t i = 0; i < n; i++) {
        const double d = fabs((double)got[i] - (double)want[i]);
        if (d > worst) worst = d;
        if (fabs((double)want[i]) > scale) scale = fabs((double)want[i]);
    }
    const double rel = scale > 0 ? worst / scale : worst;
    printf("%-28s rel err %.2e %s\n", what, rel, rel <= 1e-5 ? "ok" : "MISMATCH");
    if (!(rel <= 1e-5)) g_bad++;
}
#define CALL(expr) do { int rc__ = (expr); if (rc__ != ANE_CUDA_OK) { fprintf(stderr, "%s failed: %s\n", #expr, ane_cuda_last_error()); return 100; } } while (0)

int main(void) {
    if (ane_cuda_init(0) != ANE_CUDA_OK) { fprintf(stderr, "init: %s\n", ane_cuda_last_error()); return 99; }
    const size_t NA = (size_t)DIM * SEQ, NH = (size_t)HIDDEN * SEQ;
    const float alpha = 1.0f / sqrtf(2.0f * 12.0f);       /* train.m:188 */

    /* ---- forward: embed -> rmsnorm -> [attention] -> residual -> rmsnorm -> [FFN matmuls] -> SwiGLU -> residual -> rmsnorm */
    uint16_t *tokens = (uint16_t *)malloc(SEQ * sizeof(uint16_t)), *targets = (uint16_t *)malloc(SEQ * sizeof(uint16_t));
    int32_t *tok32 = (int32_t *)malloc(SEQ * sizeof(int32_t)), *tgt32 = (int32_t *)malloc(SEQ * sizeof(int32_t));
    for (int t = 0; t < SEQ; t++) {
        tokens[t] = (uint16_t)((t * 37 + 11) % VOCAB); targets[t] = (uint16_t)((t * 53 + 5) % VOCAB);
        tok32[t] = tokens[t]; tgt32[t] = targets[t];
    }
    tokens[7] = tokens[3];                                  /* a repeated id: its gradient rows add up in token order */
    tok32[7] = tok32[3];
    float *embed = filled((size_t)VOCAB * DIM, 0.02f), *w_att = filled(DIM, 0.02f), *w_ffn = filled(DIM, 0.02f), *w_fin = filled(DIM, 0.02f);
    for (int c = 0; c < DIM; c++) { w_att[c] += 1.0f; w_ffn[c] += 1.0f; w_fin[c] += 1.0f; }
    float *x = zeros(NA), *x_o = zeros(NA), *xn = zeros(NA), *xn_o = zeros(NA);
    CALL(ane_cuda_embed_lookup(x, embed, tokens, DIM, SEQ, VOCAB));
    orc_embed_lookup(x_o, embed, tok32, DIM, SEQ, VOCAB);
    check("embed_lookup", x, x_o, NA);
    CALL(ane_cuda_rmsnorm(xn, x, w_att, DIM, SEQ));
    orc_rmsnorm(xn_o, x, w_att, DIM, SEQ, 1e-5f);
    check("rmsnorm (attention)", xn, xn_o, NA);
    float *o_out = filled(NA, 1.0f), *x2 = zeros(NA), *x2_o = zeros(NA);           /* attention output stand-in */
    CALL(ane_cuda_residual(x2, x, o_out, alpha, NA));
    orc_residual(x2_o, x, o_out, alpha, NA);
    check("residual (attention)", x2, x2_o, NA);
    float *x2n = zeros(NA), *x2n_o = zeros(NA);
    CALL(ane_cuda_rmsnorm(x2n, x2, w_ffn, DIM, SEQ));
    orc_rmsnorm(x2n_o, x2, w_ffn, DIM, SEQ, 1e-5f);
    check("rmsnorm (FFN)", x2n, x2n_o, NA);
    float *h1 = filled(NH, 1.0f), *h3 = filled(NH, 1.0f), *gate = zeros(NH), *gate_o = zeros(NH);
    CALL(ane_cuda_swiglu(gate, h1, h3, NH));
    orc_swiglu(gate_o, h1, h3, NH);
    check("swiglu", gate, gate_o, NH);
    float *ffn = filled(NA, 1.0f), *x3 = zeros(NA), *x3_o = zeros(NA), *xf = zeros(NA), *xf_o = zeros(NA);
    CALL(ane_cuda_residual(x3, x2, ffn, alpha, NA));
    orc_residual(x3_o, x2, ffn, alpha, NA);
    check("residual (FFN)", x3, x3_o, NA);
    CALL(ane_cuda_rmsnorm(xf, x3, w_fin, DIM, SEQ));
    orc_rmsnorm(xf_o, x3, w_fin, DIM, SEQ, 1e-5f);
    check("rmsnorm (final)", xf, xf_o, NA);

    /* ---- loss */
    float *logits = filled((size_t)VOCAB * SEQ, 2.0f), *dl = zeros((size_t)VOCAB * SEQ), *dl_o = zeros((size_t)VOCAB * SEQ);
    float loss = 0.0f;
    int n_oor = 0;
    CALL(ane_cuda_cross_entropy_loss(&loss, dl, logits, targets, VOCAB, SEQ));
    const float loss_o = orc_cross_entropy(dl_o, logits, tgt32, VOCAB, SEQ, 1.0f, &n_oor);
    check("cross_entropy dlogits", dl, dl_o, (size_t)VOCAB * SEQ);
    check("cross_entropy loss", &loss, &loss_o, 1);

    /* ---- backward: rmsnorm_bwd (final) -> SwiGLU bwd -> rmsnorm_bwd (FFN) -> RoPE bwd -> rmsnorm_bwd (attention) -> embed_backward */
    float *dy = filled(NA, 1.0f), *dxf = zeros(NA), *dxf_o = zeros(NA), *dw = zeros(DIM), *dw_o = zeros(DIM);
    CALL(ane_cuda_rmsnorm_bwd(dxf, dw, dy, x3, w_fin, DIM, SEQ));
    orc_rmsnorm_bwd(dxf_o, dw_o, dy, x3, w_fin, DIM, SEQ, 1e-5f, 0);
    check("rmsnorm_bwd dx", dxf, dxf_o, NA);
    check("rmsnorm_bwd dw", dw, dw_o, DIM);
    float *dsilu = filled(NH, 1.0f), *dh1 = zeros(NH), *dh3 = zeros(NH), *dh1_o = zeros(NH), *dh3_o = zeros(NH);
    CALL(ane_cuda_swiglu_bwd(dh1, dh3, h1, h3, dsilu, NH));
    orc_swiglu_bwd(dh1_o, dh3_o, h1, h3, dsilu, NH);
    check("swiglu_bwd dh1", dh1, dh1_o, NH);
    check("swiglu_bwd dh3", dh3, dh3_o, NH);
    float *dq = filled(NA, 1.0f), *dq_o = (float *)malloc(NA * sizeof(float));
    memcpy(dq_o, dq, NA * sizeof(float));
    CALL(ane_cuda_rope_backward_inplace(dq, SEQ, DIM, HD));
    orc_rope(dq_o, SEQ, DIM, HD, 10000.0f, 0, 1);
    check("rope_backward_inplace", dq, dq_o, NA);
    float *dE = zeros((size_t)VOCAB * DIM), *dE_o = zeros((size_t)VOCAB * DIM);
    CALL(ane_cuda_embed_backward(dE, dxf, tokens, DIM, SEQ, VOCAB));
    orc_embed_backward(dE_o, dxf, tok32, DIM, SEQ, VOCAB);
    check("embed_backward", dE, dE_o, (size_t)VOCAB * DIM);

    /* ---- optimizer: both reference variants */
    const size_t NP = (size_t)VOCAB * DIM;
    float *wv = filled(NP, 0.02f), *wv_o = (float *)malloc(NP * sizeof(float)), *gr = filled(NP, 0.01f);
    memcpy(wv_o, wv, NP * sizeof(float));
    AdamState st = {zeros(NP), zeros(NP), NP};
    float *m_o = zeros(NP), *v_o = zeros(NP);
    for (int t = 1; t <= 2; t++) {
        CALL(ane_cuda_adam_update(wv, gr, &st, t, 3e-4f, 0.9f, 0.999f, 1e-8f));
        orc_adam(wv_o, gr, m_o, v_o, NP, t, 3e-4f, 0.9f, 0.999f, 1e-8f, 0.0f, 0, 1.0f, 1.0f);
    }
    check("adam_update (stories)", wv, wv_o, NP);
    for (int t = 3; t <= 4; t++) {
        CALL(ane_cuda_adam_update_wd(wv, gr, &st, t, 3e-4f, 0.9f, 0.95f, 1e-8f, 0.1f));
        orc_adam(wv_o, gr, m_o, v_o, NP, t, 3e-4f, 0.9f, 0.95f, 1e-8f, 0.1f, 1, 1.0f, 1.0f);
    }
    check("adam_update_wd (dynamic)", wv, wv_o, NP);
    check("adam moments m", st.m, m_o, NP);
    check("adam moments v", st.v, v_o, NP);

    ane_cuda_status stw;
    ane_cuda_poll_status(&stw, 1);
    printf("status: out-of-range ids %d, non-finite losses %d; %lld kernel launches\n", stw.oor_ids, stw.nonfinite, ane_cuda_launch_count());
    ane_cuda_shutdown();
    printf(g_bad ? "%d operator(s) disagree with the oracle\n" : "all operators agree with the oracle\n", g_bad);
    return g_bad;
}
