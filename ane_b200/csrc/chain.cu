// chain.cu -- the operator chain of one micro-batch with HOST buffers on the contraction side, for a C caller.
//
// In the reference's loop the contractions (QKV / output / FFN projections, SDPA, classifier) run on another engine
// and hand their results over in host memory; everything between them is this library's operator set
// (training_dynamic/train.m:428-482 forward, :527-720 backward).  ane_cuda_chain_step is that arrangement end to
// end: per layer it copies what the contractions produced host -> device, runs the operators in the order of the
// reference's loop, and copies what the next contraction consumes device -> host -- on three streams (upload,
// operators, download), so that the copies of one layer overlap the operators of its neighbours, which one blocking
// ane_cuda_*_host call per operator cannot do.  Tensors only the operators consume (the residual stream, x2, the
// running gradient) never leave the device.
//
// The operators are the library's own device entry points, called in the same order with the same arguments as
// ane_b200/layer_chain.py does, so both give the same bits.
#include "common.cuh"

#include <vector>

using namespace ane;

struct ANECudaChain {
    ane_chain_config c;
    ane_chain_params p;
    int B = 0, R = 0;
    size_t e = 2;
    std::vector<void *> owned;                       // every device allocation of the chain
    // per layer: device copies of the contraction outputs (kept for the backward pass) and the chain's own saves
    std::vector<void *> q, k, o_out, h1, h3, ffn_out, layer_in, x2;
    // rotating sets
    std::vector<void *> xnorm, q_r, k_r, x2norm, gate, dsilu, dx_ffn, dq_in, dk_in, dx_attn, dh1, dh3, dq, dk;
    void *x_final = nullptr, *dy_cls = nullptr, *dy[2] = {nullptr, nullptr}, *dx2 = nullptr;
    int32_t *tokens = nullptr;
    cudaStream_t s_in = nullptr, s_c = nullptr, s_out = nullptr;
    std::vector<cudaEvent_t> e_in_f, e_c_f, e_out_f, e_in_b, e_c_b, e_out_b;
    cudaEvent_t e_misc_in = nullptr, e_fwd_done = nullptr, e_step_done = nullptr;
    bool first = true;
    size_t bytes(int channels) const { return (size_t)B * channels * c.seq * e; }
};

namespace ane {

static bool chain_alloc(ANECudaChain *ch, void **out, size_t bytes) {
    void *p = nullptr;
    if (dev_malloc(&p, bytes) != cudaSuccess) return false;
    ch->owned.push_back(p);
    *out = p;
    return true;
}

static bool chain_alloc_set(ANECudaChain *ch, std::vector<void *> &v, int count, int channels) {
    v.resize(count);
    for (int i = 0; i < count; i++)
        if (!chain_alloc(ch, &v[i], ch->bytes(channels))) return false;
    return true;
}

static void chain_free(ANECudaChain *ch) {
    if (!ch) return;
    cudaDeviceSynchronize();
    for (void *p : ch->owned) cudaFree(p);
    for (auto *v : {&ch->e_in_f, &ch->e_c_f, &ch->e_out_f, &ch->e_in_b, &ch->e_c_b, &ch->e_out_b})
        for (cudaEvent_t ev : *v) if (ev) cudaEventDestroy(ev);
    for (cudaEvent_t ev : {ch->e_misc_in, ch->e_fwd_done, ch->e_step_done}) if (ev) cudaEventDestroy(ev);
    for (cudaStream_t s : {ch->s_in, ch->s_c, ch->s_out}) if (s) cudaStreamDestroy(s);
    delete ch;
}

#define CH_TRY(expr) do { if (int rc__ = (expr)) return rc__; } while (0)

static int chain_fwd_begin(ANECudaChain *ch) {
    const auto &c = ch->c;
    CH_TRY(ane_cuda_embed_lookup_dev(ch->s_c, c.dtype, ANE_ID_I32, ch->B, c.dim, c.seq, ch->layer_in[0], ch->p.table, ch->tokens, c.vocab, ANE_OOR_SKIP));
    return ane_cuda_rmsnorm_dev(ch->s_c, c.dtype, ch->B, c.dim, c.seq, ch->xnorm[0], ch->layer_in[0], ch->p.att_w, c.eps);
}

static int chain_fwd_layer(ANECudaChain *ch, int l) {
    const auto &c = ch->c;
    const auto &p = ch->p;
    const int r = l % ch->R, B = ch->B;
    CH_TRY(ane_cuda_qknorm_rope_pair_dev(ch->s_c, c.dtype, B, c.heads, c.kv_heads, c.head_dim, c.seq, ch->q_r[r], ch->k_r[r], ch->q[l], ch->k[l],
                                         p.q_w + (size_t)l * c.head_dim, p.k_w + (size_t)l * c.head_dim, c.qk_eps, c.rope_base, 0));
    CH_TRY(ane_cuda_residual_rmsnorm_dev(ch->s_c, c.dtype, B, c.dim, c.seq, ch->x2[l], ch->x2norm[r], ch->layer_in[l], ch->o_out[l],
                                         p.ffn_w + (size_t)l * c.dim, c.alpha, c.eps));                                     // train.m:460-461
    CH_TRY(ane_cuda_swiglu_dev(ch->s_c, c.dtype, (size_t)B * c.hidden * c.seq, ch->gate[r], ch->h1[l], ch->h3[l]));
    // x_next = x2 + alpha * ffn (train.m:497) fused with the norm that reads it next
    const bool last = l + 1 == c.layers;
    const float *w_next = last ? p.final_w : p.att_w + (size_t)(l + 1) * c.dim;
    void *n_next = last ? ch->x_final : ch->xnorm[(l + 1) % ch->R];
    return ane_cuda_residual_rmsnorm_dev(ch->s_c, c.dtype, B, c.dim, c.seq, ch->layer_in[l + 1], n_next, ch->x2[l], ch->ffn_out[l], w_next, c.alpha, c.eps);
}

static int chain_bwd_layer(ANECudaChain *ch, int l, int &cur) {
    const auto &c = ch->c;
    const auto &p = ch->p;
    const int r = l % ch->R, B = ch->B;
    void *dyc = ch->dy[cur], *nxt = ch->dy[1 - cur];
    CH_TRY(ane_cuda_swiglu_bwd_dev(ch->s_c, c.dtype, (size_t)B * c.hidden * c.seq, ch->dh1[r], ch->dh3[r], ch->h1[l], ch->h3[l], ch->dsilu[r]));   // train.m:537-554
    CH_TRY(ane_cuda_rmsnorm_bwd_dev(ch->s_c, c.dtype, B, c.dim, c.seq, ch->dx2, p.ffn_g + (size_t)l * c.dim, ch->dx_ffn[r], ch->x2[l],
                                    p.ffn_w + (size_t)l * c.dim, dyc, c.eps, c.norm_bwd_flags));                             // train.m:588-590
    CH_TRY(ane_cuda_rope_qknorm_bwd_pair_dev(ch->s_c, c.dtype, B, c.heads, c.kv_heads, c.head_dim, c.seq, ch->dq[r], ch->dk[r],
                                             p.q_g + (size_t)l * c.head_dim, p.k_g + (size_t)l * c.head_dim, ch->dq_in[r], ch->dk_in[r], ch->q[l], ch->k[l],
                                             p.q_w + (size_t)l * c.head_dim, p.k_w + (size_t)l * c.head_dim, c.qk_eps, c.rope_base, 0, c.norm_bwd_flags));
    CH_TRY(ane_cuda_rmsnorm_bwd_dev(ch->s_c, c.dtype, B, c.dim, c.seq, nxt, p.att_g + (size_t)l * c.dim, ch->dx_attn[r], ch->layer_in[l],
                                    p.att_w + (size_t)l * c.dim, ch->dx2, c.eps, c.norm_bwd_flags));                         // train.m:719-722
    cur = 1 - cur;
    return ANE_CUDA_OK;
}

static int copy_async(void *dst, const void *src, size_t bytes, cudaMemcpyKind kind, cudaStream_t st) {
    ANE_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, kind, st));
    return ANE_CUDA_OK;
}

}  // namespace ane

extern "C" {

ANECudaChain *ane_cuda_chain_create(const ane_chain_config *cfg, int n_seqs, const ane_chain_params *params) {
    if (!ctx().inited) { fail(ANE_CUDA_ERR_NOT_INIT, "%s: call ane_cuda_init first", __func__); return nullptr; }
    if (!cfg || !params || n_seqs < 1) { fail(ANE_CUDA_ERR_INVALID, "%s: null pointer or no sequences", __func__); return nullptr; }
    const ane_chain_config &c = *cfg;
    if (c.layers < 1 || c.dim < 1 || c.hidden < 1 || c.heads < 1 || c.kv_heads < 1 || c.head_dim < 2 || c.seq < 1 || c.vocab < 1 ||
        !dtype_ok(c.dtype) || c.rotate < 1 ||
        (c.norm_bwd_flags != ANE_NORM_BWD_REFERENCE && c.norm_bwd_flags != ANE_NORM_BWD_EXACT)) {
        fail(ANE_CUDA_ERR_INVALID, "%s: bad configuration", __func__);
        return nullptr;
    }
    const ane_chain_params &p = *params;
    if (!p.att_w || !p.ffn_w || !p.final_w || !p.q_w || !p.k_w || !p.att_g || !p.ffn_g || !p.final_g || !p.q_g || !p.k_g || !p.table || !p.embed_g) {
        fail(ANE_CUDA_ERR_INVALID, "%s: a parameter pointer is null", __func__);
        return nullptr;
    }
    ANECudaChain *ch = new ANECudaChain();
    ch->c = c;
    ch->p = p;
    ch->B = n_seqs;
    ch->R = c.rotate;
    ch->e = dtype_size(c.dtype);
    const int L = c.layers, R = c.rotate, qd = c.heads * c.head_dim, kvd = c.kv_heads * c.head_dim;
    bool ok = chain_alloc_set(ch, ch->q, L, qd) && chain_alloc_set(ch, ch->k, L, kvd) && chain_alloc_set(ch, ch->o_out, L, c.dim) &&
              chain_alloc_set(ch, ch->h1, L, c.hidden) && chain_alloc_set(ch, ch->h3, L, c.hidden) && chain_alloc_set(ch, ch->ffn_out, L, c.dim) &&
              chain_alloc_set(ch, ch->layer_in, L + 1, c.dim) && chain_alloc_set(ch, ch->x2, L, c.dim) &&
              chain_alloc_set(ch, ch->xnorm, R, c.dim) && chain_alloc_set(ch, ch->q_r, R, qd) && chain_alloc_set(ch, ch->k_r, R, kvd) &&
              chain_alloc_set(ch, ch->x2norm, R, c.dim) && chain_alloc_set(ch, ch->gate, R, c.hidden) &&
              chain_alloc_set(ch, ch->dsilu, R, c.hidden) && chain_alloc_set(ch, ch->dx_ffn, R, c.dim) && chain_alloc_set(ch, ch->dq_in, R, qd) &&
              chain_alloc_set(ch, ch->dk_in, R, kvd) && chain_alloc_set(ch, ch->dx_attn, R, c.dim) && chain_alloc_set(ch, ch->dh1, R, c.hidden) &&
              chain_alloc_set(ch, ch->dh3, R, c.hidden) && chain_alloc_set(ch, ch->dq, R, qd) && chain_alloc_set(ch, ch->dk, R, kvd) &&
              chain_alloc(ch, &ch->x_final, ch->bytes(c.dim)) && chain_alloc(ch, &ch->dy_cls, ch->bytes(c.dim)) &&
              chain_alloc(ch, &ch->dy[0], ch->bytes(c.dim)) && chain_alloc(ch, &ch->dy[1], ch->bytes(c.dim)) &&
              chain_alloc(ch, &ch->dx2, ch->bytes(c.dim)) && chain_alloc(ch, reinterpret_cast<void **>(&ch->tokens), (size_t)n_seqs * c.seq * sizeof(int32_t));
    if (!ok) {
        fail(ANE_CUDA_ERR_NOMEM, "%s: not enough device memory for %d sequences x %d layers", __func__, n_seqs, L);
        chain_free(ch);
        return nullptr;
    }
    auto stream = [&](cudaStream_t *s) { return cudaStreamCreateWithFlags(s, cudaStreamNonBlocking) == cudaSuccess; };
    auto event = [&](cudaEvent_t *ev) { return cudaEventCreateWithFlags(ev, cudaEventDisableTiming) == cudaSuccess; };
    ok = stream(&ch->s_in) && stream(&ch->s_c) && stream(&ch->s_out) && event(&ch->e_misc_in) && event(&ch->e_fwd_done) && event(&ch->e_step_done);
    for (auto *v : {&ch->e_in_f, &ch->e_c_f, &ch->e_out_f, &ch->e_in_b, &ch->e_c_b, &ch->e_out_b}) {
        v->assign(L, nullptr);
        for (int l = 0; l < L && ok; l++) ok = event(&(*v)[l]);
    }
    if (!ok) {
        cudaGetLastError();
        fail(ANE_CUDA_ERR_CUDA, "%s: cannot create streams and events", __func__);
        chain_free(ch);
        return nullptr;
    }
    return ch;
}

void ane_cuda_chain_destroy(ANECudaChain *ch) { chain_free(ch); }

size_t ane_cuda_chain_h2d_bytes(const ANECudaChain *ch) {
    if (!ch) return 0;
    const auto &c = ch->c;
    const size_t qd = (size_t)c.heads * c.head_dim, kvd = (size_t)c.kv_heads * c.head_dim, T = (size_t)ch->B * c.seq;
    const size_t per_layer = qd + kvd + c.dim + 2 * (size_t)c.hidden + c.dim + c.hidden + c.dim + qd + kvd + c.dim;
    return T * ch->e * ((size_t)c.layers * per_layer + c.dim) + T * 4;
}

size_t ane_cuda_chain_d2h_bytes(const ANECudaChain *ch) {
    if (!ch) return 0;
    const auto &c = ch->c;
    const size_t qd = (size_t)c.heads * c.head_dim, kvd = (size_t)c.kv_heads * c.head_dim, T = (size_t)ch->B * c.seq;
    const size_t per_layer = c.dim + qd + kvd + c.dim + c.hidden + 2 * (size_t)c.hidden + qd + kvd;
    return T * ch->e * ((size_t)c.layers * per_layer + c.dim);
}

int ane_cuda_chain_step(ANECudaChain *ch, const ane_chain_host_io *io) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(ch && io, "%s: null pointer", __func__);
    ANE_REQUIRE(io->q && io->k && io->o_out && io->h1 && io->h3 && io->ffn_out && io->xnorm && io->q_r && io->k_r && io->x2norm && io->gate &&
                io->dsilu && io->dx_ffn && io->dq_in && io->dk_in && io->dx_attn && io->dh1 && io->dh3 && io->dq && io->dk && io->dy_cls &&
                io->x_final && io->tokens, "%s: a host pointer table is null", __func__);
    const auto &c = ch->c;
    const int L = c.layers, R = ch->R;
    const int qd = c.heads * c.head_dim, kvd = c.kv_heads * c.head_dim;
    const size_t bD = ch->bytes(c.dim), bH = ch->bytes(c.hidden), bQ = ch->bytes(qd), bK = ch->bytes(kvd);
    for (int l = 0; l < L; l++)
        ANE_REQUIRE(io->q[l] && io->k[l] && io->o_out[l] && io->h1[l] && io->h3[l] && io->ffn_out[l] && io->xnorm[l] && io->q_r[l] && io->k_r[l] &&
                    io->x2norm[l] && io->gate[l] && io->dsilu[l] && io->dx_ffn[l] && io->dq_in[l] && io->dk_in[l] && io->dx_attn[l] && io->dh1[l] &&
                    io->dh3[l] && io->dq[l] && io->dk[l], "%s: a host buffer of layer %d is null", __func__, l);
    cudaStream_t s_in = ch->s_in, s_c = ch->s_c, s_out = ch->s_out;
    const cudaMemcpyKind H2D = cudaMemcpyHostToDevice, D2H = cudaMemcpyDeviceToHost;

    // ---- forward: uploads of all layers are enqueued first; the operators of layer l wait for its upload only
    if (!ch->first) ANE_CUDA_TRY(cudaStreamWaitEvent(s_in, ch->e_step_done, 0));      // last step's operators still read the per-layer inputs
    CH_TRY(copy_async(ch->tokens, io->tokens, (size_t)ch->B * c.seq * sizeof(int32_t), H2D, s_in));
    CH_TRY(copy_async(ch->dy_cls, io->dy_cls, bD, H2D, s_in));
    ANE_CUDA_TRY(cudaEventRecord(ch->e_misc_in, s_in));
    for (int l = 0; l < L; l++) {
        CH_TRY(copy_async(ch->q[l], io->q[l], bQ, H2D, s_in));
        CH_TRY(copy_async(ch->k[l], io->k[l], bK, H2D, s_in));
        CH_TRY(copy_async(ch->o_out[l], io->o_out[l], bD, H2D, s_in));
        CH_TRY(copy_async(ch->h1[l], io->h1[l], bH, H2D, s_in));
        CH_TRY(copy_async(ch->h3[l], io->h3[l], bH, H2D, s_in));
        CH_TRY(copy_async(ch->ffn_out[l], io->ffn_out[l], bD, H2D, s_in));
        ANE_CUDA_TRY(cudaEventRecord(ch->e_in_f[l], s_in));
    }
    ANE_CUDA_TRY(cudaStreamWaitEvent(s_c, ch->e_misc_in, 0));
    CH_TRY(chain_fwd_begin(ch));                                                         // gather + the first layer's attention norm
    ANE_CUDA_TRY(cudaEventRecord(ch->e_fwd_done, s_c));
    ANE_CUDA_TRY(cudaStreamWaitEvent(s_out, ch->e_fwd_done, 0));
    CH_TRY(copy_async(io->xnorm[0], ch->xnorm[0], bD, D2H, s_out));
    for (int l = 0; l < L; l++) {
        ANE_CUDA_TRY(cudaStreamWaitEvent(s_c, ch->e_in_f[l], 0));
        if (l >= R) ANE_CUDA_TRY(cudaStreamWaitEvent(s_c, ch->e_out_f[l - R], 0));       // the rotating outputs of layer l-R have left the device
        CH_TRY(chain_fwd_layer(ch, l));
        ANE_CUDA_TRY(cudaEventRecord(ch->e_c_f[l], s_c));
        ANE_CUDA_TRY(cudaStreamWaitEvent(s_out, ch->e_c_f[l], 0));
        const int r = l % R;
        CH_TRY(copy_async(io->q_r[l], ch->q_r[r], bQ, D2H, s_out));
        CH_TRY(copy_async(io->k_r[l], ch->k_r[r], bK, D2H, s_out));
        CH_TRY(copy_async(io->x2norm[l], ch->x2norm[r], bD, D2H, s_out));
        CH_TRY(copy_async(io->gate[l], ch->gate[r], bH, D2H, s_out));
        if (l + 1 < L) CH_TRY(copy_async(io->xnorm[l + 1], ch->xnorm[(l + 1) % R], bD, D2H, s_out));   // layer l closes with the next layer's norm
        ANE_CUDA_TRY(cudaEventRecord(ch->e_out_f[l], s_out));
    }
    ANE_CUDA_TRY(cudaEventRecord(ch->e_fwd_done, s_c));
    ANE_CUDA_TRY(cudaStreamWaitEvent(s_out, ch->e_fwd_done, 0));
    CH_TRY(copy_async(io->x_final, ch->x_final, bD, D2H, s_out));

    // ---- backward, layers in reverse
    CH_TRY(ane_cuda_rmsnorm_bwd_dev(s_c, c.dtype, ch->B, c.dim, c.seq, ch->dy[0], ch->p.final_g, ch->dy_cls, ch->layer_in[L], ch->p.final_w, nullptr,
                                    c.eps, c.norm_bwd_flags));
    int cur = 0;
    for (int i = 0; i < L; i++) {
        const int l = L - 1 - i, r = l % R;
        if (i >= R) ANE_CUDA_TRY(cudaStreamWaitEvent(s_in, ch->e_c_b[L - 1 - (i - R)], 0));   // the rotating inputs of that layer have been consumed
        CH_TRY(copy_async(ch->dsilu[r], io->dsilu[l], bH, H2D, s_in));
        CH_TRY(copy_async(ch->dx_ffn[r], io->dx_ffn[l], bD, H2D, s_in));
        CH_TRY(copy_async(ch->dq_in[r], io->dq_in[l], bQ, H2D, s_in));
        CH_TRY(copy_async(ch->dk_in[r], io->dk_in[l], bK, H2D, s_in));
        CH_TRY(copy_async(ch->dx_attn[r], io->dx_attn[l], bD, H2D, s_in));
        ANE_CUDA_TRY(cudaEventRecord(ch->e_in_b[l], s_in));
        ANE_CUDA_TRY(cudaStreamWaitEvent(s_c, ch->e_in_b[l], 0));
        if (i >= R) ANE_CUDA_TRY(cudaStreamWaitEvent(s_c, ch->e_out_b[L - 1 - (i - R)], 0));  // the rotating outputs of that layer have left the device
        CH_TRY(chain_bwd_layer(ch, l, cur));
        ANE_CUDA_TRY(cudaEventRecord(ch->e_c_b[l], s_c));
        ANE_CUDA_TRY(cudaStreamWaitEvent(s_out, ch->e_c_b[l], 0));
        CH_TRY(copy_async(io->dh1[l], ch->dh1[r], bH, D2H, s_out));
        CH_TRY(copy_async(io->dh3[l], ch->dh3[r], bH, D2H, s_out));
        CH_TRY(copy_async(io->dq[l], ch->dq[r], bQ, D2H, s_out));
        CH_TRY(copy_async(io->dk[l], ch->dk[r], bK, D2H, s_out));
        ANE_CUDA_TRY(cudaEventRecord(ch->e_out_b[l], s_out));
    }
    CH_TRY(ane_cuda_embed_backward_dev(s_c, c.dtype, ANE_ID_I32, ch->B, c.dim, c.seq, ch->p.embed_g, ch->dy[cur], ch->tokens, c.vocab));
    ANE_CUDA_TRY(cudaEventRecord(ch->e_step_done, s_c));
    ch->first = false;
    return ANE_CUDA_OK;
}

int ane_cuda_chain_sync(ANECudaChain *ch) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(ch, "%s: null pointer", __func__);
    ANE_CUDA_TRY(cudaStreamSynchronize(ch->s_in));
    ANE_CUDA_TRY(cudaStreamSynchronize(ch->s_c));
    ANE_CUDA_TRY(cudaStreamSynchronize(ch->s_out));
    return ANE_CUDA_OK;
}

void *ane_cuda_chain_compute_stream(ANECudaChain *ch) { return ch ? (void *)ch->s_c : nullptr; }

}  // extern "C"
