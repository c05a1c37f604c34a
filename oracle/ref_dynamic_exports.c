/* Exported wrappers around the `static` functions of the reference's
 * training/training_dynamic/cpu_ops.h (compiled from standard input, see
 * ref_stories_exports.c).  TEST INFRASTRUCTURE ONLY.
 * The header keeps a file-scope scratch row sized by the first call's S
 * (cpu_ops.h:5,8,25); ref_dynamic_reset() frees it so one process can use several S. */
void ref_dynamic_reset(void) { if (g_rms_tmp) { free(g_rms_tmp); g_rms_tmp = NULL; } }
void ref_dynamic_rmsnorm(float *out, const float *x, const float *w, int d, int S) {
    ref_dynamic_reset(); rmsnorm(out, x, w, d, S);
}
void ref_dynamic_rmsnorm_bwd(float *dx, float *dw, const float *dy, const float *x, const float *w, int d, int S) {
    ref_dynamic_reset(); rmsnorm_bwd(dx, dw, dy, x, w, d, S);
}
void ref_dynamic_adam_update(float *w, const float *g, float *m, float *v, size_t n, int t,
                             float lr, float b1, float b2, float eps, float wd) {
    AdamState s; s.m = m; s.v = v; s.n = n;
    adam_update(w, g, &s, t, lr, b1, b2, eps, wd);
}
float ref_dynamic_cross_entropy_loss(float *dlogits, const float *logits, const uint16_t *targets, int V, int S) {
    return cross_entropy_loss(dlogits, logits, targets, V, S);
}
void ref_dynamic_embed_lookup(float *x, const float *embed, const uint16_t *tokens, int dim, int seq) {
    embed_lookup(x, embed, tokens, dim, seq);
}
void ref_dynamic_embed_backward(float *d_embed, const float *dx, const uint16_t *tokens, int dim, int seq) {
    embed_backward(d_embed, dx, tokens, dim, seq);
}
void ref_dynamic_rope_backward_inplace(float *dx, int seq, int dim, int hd) {
    rope_backward_inplace(dx, seq, dim, hd);
}
/* Vocab compaction helpers (cpu_ops.h:96-148). */
int ref_dynamic_vocab_map_build(const uint16_t *data, size_t n_tokens, int full_vocab,
                                int *full_to_compact, int *compact_to_full) {
    VocabMap vm = vocab_map_build(data, n_tokens, full_vocab);
    memcpy(full_to_compact, vm.full_to_compact, (size_t)full_vocab * sizeof(int));
    memcpy(compact_to_full, vm.compact_to_full, (size_t)vm.compact_vocab * sizeof(int));
    int cv = vm.compact_vocab;
    free(vm.full_to_compact); free(vm.compact_to_full);
    return cv;
}

void ref_dynamic_vocab_compact_embed(float *compact, const float *full_embed, const int *compact_to_full, int compact_vocab, int dim) {
    VocabMap vm = {compact_vocab, NULL, (int *)compact_to_full};
    float *ce = vocab_compact_embed(full_embed, &vm, dim);
    memcpy(compact, ce, (size_t)compact_vocab * dim * 4);
    free(ce);
}
void ref_dynamic_vocab_scatter_grads(float *full_gembed, const float *compact_gembed, const int *compact_to_full, int compact_vocab, int dim) {
    VocabMap vm = {compact_vocab, NULL, (int *)compact_to_full};
    vocab_scatter_grads(full_gembed, compact_gembed, &vm, dim);
}
void ref_dynamic_vocab_update_full(float *full_embed, const float *compact_embed, const int *compact_to_full, int compact_vocab, int dim) {
    VocabMap vm = {compact_vocab, NULL, (int *)compact_to_full};
    vocab_update_full(full_embed, compact_embed, &vm, dim);
}
