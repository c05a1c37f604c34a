/* Exported wrappers around the `static` functions of the reference's
 * training/stories_cpu_ops.h.  The build recipe (build_oracle.py) feeds the compiler
 *     <reference header text> + <this file>
 * on standard input, so the reference source is compiled from where it lies and is never
 * copied into this repository.  TEST INFRASTRUCTURE ONLY. */
int g_ref_vocab = 32000;
void ref_stories_set_vocab(int v) { g_ref_vocab = v; }
void ref_stories_rmsnorm(float *out, const float *x, const float *w, int d, int S) { rmsnorm(out, x, w, d, S); }
void ref_stories_rmsnorm_bwd(float *dx, float *dw, const float *dy, const float *x, const float *w, int d, int S) {
    rmsnorm_bwd(dx, dw, dy, x, w, d, S);
}
void ref_stories_adam_update(float *w, const float *g, float *m, float *v, size_t n, int t,
                             float lr, float b1, float b2, float eps) {
    AdamState s; s.m = m; s.v = v; s.n = n;
    adam_update(w, g, &s, t, lr, b1, b2, eps);
}
float ref_stories_cross_entropy_loss(float *dlogits, const float *logits, const uint16_t *targets, int V, int S) {
    return cross_entropy_loss(dlogits, logits, targets, V, S);
}
void ref_stories_embed_lookup(float *x, const float *embed, const uint16_t *tokens, int dim, int seq) {
    embed_lookup(x, embed, tokens, dim, seq);
}
void ref_stories_embed_backward(float *d_embed, const float *dx, const uint16_t *tokens, int dim, int seq) {
    embed_backward(d_embed, dx, tokens, dim, seq);
}
