// ckpt.cu -- reader / writer of the reference's training checkpoints ("BLZT" files) straight to and from
// the flat device buffers the optimizer works on.  Host-side code only (file I/O and copies).
//
// File layout (training/train_large.m:109-145 version 2, training_dynamic/train.m:104-138 version 4):
//   header, 96 bytes (stories_config.h:95-104 / training_dynamic/config.h:78-86)
//   per layer:  Wq Wk Wv Wo W1 W2 W3 rms_att rms_ffn            (fp32 weights)
//               then (m, v) of each of the nine, in the same order (Adam moments)
//   rms_final, its m, its v;  embed [vocab][dim], its m, its v
// Version 2 has square attention matrices (Wq = Wk = Wv = Wo = dim x dim); version 4 stores
// kv_heads / head_dim / q_dim where version 2 has padding, and Wk, Wv are kv_dim x dim.
//
// Device layout ("weight order"): the weights in file order with the moments taken out --
//   [layer 0: Wq Wk Wv Wo W1 W2 W3 rms_att rms_ffn] ... [layer L-1: ...] rms_final embed
// -- in three parallel buffers w, m, v of ane_cuda_ckpt_param_count() floats each.
//
// Device layout ("optimizer order", the *_flat entry points): what a flat optimizer wants -- everything that takes
// weight decay first, the norm weights (no decay, train.m:837-869) after it:
//   [layer 0: Wq Wk Wv Wo W1 W2 W3] ... [layer L-1: ...] embed | rms_att[0..L-1] rms_ffn[0..L-1] rms_final | (caller's extras)
// The first ane_cuda_ckpt_flat_decay_count() floats are the decayed range; floats beyond param_count (for example
// per-head QK-norm weights, which the reference's files do not store) are left untouched by a load and are not
// written by a save.
//
// llama2.c weight files (train_large.m:13-56): a 7-int header, then embed, rms_att[all layers], wq[all], wk[all],
// wv[all], wo[all], rms_ffn[all], w1[all], w2[all], w3[all], rms_final (then RoPE tables and, when vocab_size < 0, a
// separate classifier, neither of which the reference reads).
#include "common.cuh"

#include <stdio.h>
#include <string.h>

#include <vector>

namespace ane {

constexpr int CKPT_MAGIC = 0x424C5A54;     // "BLZT"

struct Extent { size_t count; };

// sizes of the nine per-layer tensors, in file order
static bool layer_extents(const ane_ckpt_header &h, size_t (&sz)[9]) {
    if (h.n_layers < 1 || h.dim < 1 || h.hidden_dim < 1 || h.vocab_size < 1) return false;
    size_t q_dim = (size_t)h.dim, kv_dim = (size_t)h.dim;
    if (h.version >= 4) {
        if (h.kv_heads < 1 || h.head_dim < 1 || h.q_dim < 1) return false;
        q_dim = (size_t)h.q_dim;
        kv_dim = (size_t)h.kv_heads * h.head_dim;
    }
    const size_t d = (size_t)h.dim, hid = (size_t)h.hidden_dim;
    sz[0] = q_dim * d;  sz[1] = kv_dim * d;  sz[2] = kv_dim * d;  sz[3] = d * q_dim;     // Wq Wk Wv Wo
    sz[4] = hid * d;    sz[5] = d * hid;     sz[6] = hid * d;                             // W1 W2 W3
    sz[7] = d;          sz[8] = d;                                                        // rms_att rms_ffn
    return true;
}

static size_t param_count(const ane_ckpt_header &h) {
    size_t sz[9];
    if (!layer_extents(h, sz)) return 0;
    size_t per_layer = 0;
    for (int i = 0; i < 9; i++) per_layer += sz[i];
    return per_layer * h.n_layers + (size_t)h.dim + (size_t)h.vocab_size * h.dim;
}

static int read_header(FILE *f, ane_ckpt_header *h) {
    if (fread(h, sizeof(*h), 1, f) != 1) return fail(ANE_CUDA_ERR_INVALID, "checkpoint: file shorter than its header");
    if (h->magic != CKPT_MAGIC) return fail(ANE_CUDA_ERR_INVALID, "checkpoint: bad magic 0x%08x", (unsigned)h->magic);
    if (h->version != 2 && h->version != 4) return fail(ANE_CUDA_ERR_INVALID, "checkpoint: unsupported version %d", h->version);
    if (param_count(*h) == 0) return fail(ANE_CUDA_ERR_INVALID, "checkpoint: inconsistent dimensions in the header");
    return ANE_CUDA_OK;
}

enum Layout { WEIGHT_ORDER = 0, OPTIMIZER_ORDER = 1 };
enum Tensor { T_WQ = 0, T_WK, T_WV, T_WO, T_W1, T_W2, T_W3, T_RMS_ATT, T_RMS_FFN, T_RMS_FINAL, T_EMBED };

// Offset (in floats) of tensor `t` of layer `L` in a device buffer of the given layout.
static size_t tensor_offset(const ane_ckpt_header &h, Layout layout, int t, int L) {
    size_t sz[9];
    layer_extents(h, sz);
    size_t per_layer = 0, matrices = 0;
    for (int i = 0; i < 9; i++) { per_layer += sz[i]; if (i < 7) matrices += sz[i]; }
    const size_t nl = (size_t)h.n_layers, d = (size_t)h.dim, e = (size_t)h.vocab_size * h.dim;
    size_t within = 0;
    if (t < 9) for (int i = 0; i < t; i++) within += sz[i];
    if (layout == WEIGHT_ORDER) {
        if (t < 9) return (size_t)L * per_layer + within;
        return nl * per_layer + (t == T_EMBED ? d : 0);
    }
    if (t < 7) return (size_t)L * matrices + within;
    if (t == T_EMBED) return nl * matrices;
    const size_t norms = nl * matrices + e;
    if (t == T_RMS_ATT) return norms + (size_t)L * d;
    if (t == T_RMS_FFN) return norms + nl * d + (size_t)L * d;
    return norms + 2 * nl * d;                                                           // rms_final
}

// One pass over the file's tensors in file order.  io(dev_buffer_index 0/1/2 = w/m/v, offset in floats, count) moves
// `count` floats between the file position and the device range.
template <class IO>
static int walk(const ane_ckpt_header &h, Layout layout, IO io) {
    size_t sz[9];
    layer_extents(h, sz);
    for (int L = 0; L < h.n_layers; L++) {
        for (int i = 0; i < 9; i++) if (int rc = io(0, tensor_offset(h, layout, i, L), sz[i])) return rc;
        for (int i = 0; i < 9; i++) {
            if (int rc = io(1, tensor_offset(h, layout, i, L), sz[i])) return rc;
            if (int rc = io(2, tensor_offset(h, layout, i, L), sz[i])) return rc;
        }
    }
    const size_t d = (size_t)h.dim, e = (size_t)h.vocab_size * h.dim;
    for (int which = 0; which < 3; which++) if (int rc = io(which, tensor_offset(h, layout, T_RMS_FINAL, 0), d)) return rc;
    for (int which = 0; which < 3; which++) if (int rc = io(which, tensor_offset(h, layout, T_EMBED, 0), e)) return rc;
    return ANE_CUDA_OK;
}

constexpr size_t CKPT_CHUNK = (size_t)8 << 20;      // floats per staging chunk (32 MiB)

}  // namespace ane

using namespace ane;

extern "C" {

int ane_cuda_ckpt_read_header(const char *path, ane_ckpt_header *hdr) {
    ANE_REQUIRE(path && hdr, "%s: null pointer", __func__);
    FILE *f = fopen(path, "rb");
    if (!f) return fail(ANE_CUDA_ERR_INVALID, "%s: cannot open %s", __func__, path);
    const int rc = read_header(f, hdr);
    fclose(f);
    return rc;
}

size_t ane_cuda_ckpt_param_count(const ane_ckpt_header *hdr) { return hdr ? param_count(*hdr) : 0; }

static int ckpt_load(Layout layout, const char *path, ane_ckpt_header *hdr, float *w_dev, float *m_dev, float *v_dev,
                     size_t n_floats) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(path && hdr && w_dev, "%s: null pointer", __func__);
    ANE_REQUIRE((m_dev == nullptr) == (v_dev == nullptr), "%s: give both moment buffers or neither", __func__);
    FILE *f = fopen(path, "rb");
    if (!f) return fail(ANE_CUDA_ERR_INVALID, "%s: cannot open %s", __func__, path);
    int rc = read_header(f, hdr);
    if (rc == ANE_CUDA_OK && (layout == WEIGHT_ORDER ? param_count(*hdr) != n_floats : param_count(*hdr) > n_floats))
        rc = fail(ANE_CUDA_ERR_INVALID, "%s: the file holds %zu parameters, the buffers %zu", __func__, param_count(*hdr), n_floats);
    if (rc == ANE_CUDA_OK) {      // the whole body must be there, also the parts a weights-only load skips over
        const long body = (long)sizeof(*hdr);
        if (fseek(f, 0, SEEK_END) != 0 || ftell(f) < 0 || (size_t)ftell(f) < sizeof(*hdr) + 3 * sizeof(float) * param_count(*hdr))
            rc = fail(ANE_CUDA_ERR_INVALID, "%s: %s is truncated (%ld bytes, the header promises %zu)", __func__, path, ftell(f),
                      sizeof(*hdr) + 3 * sizeof(float) * param_count(*hdr));
        else if (fseek(f, body, SEEK_SET) != 0)
            rc = fail(ANE_CUDA_ERR_INVALID, "%s: seek failed", __func__);
    }
    if (rc != ANE_CUDA_OK) { fclose(f); return rc; }
    std::vector<float> stage(CKPT_CHUNK);
    float *dst[3] = {w_dev, m_dev, v_dev};
    rc = walk(*hdr, layout, [&](int which, size_t off, size_t count) -> int {
        if (!dst[which]) return fseek(f, (long)(count * sizeof(float)), SEEK_CUR) == 0 ? ANE_CUDA_OK
                                                                                        : fail(ANE_CUDA_ERR_INVALID, "%s: seek failed", __func__);
        for (size_t done = 0; done < count; done += CKPT_CHUNK) {
            const size_t n = count - done < CKPT_CHUNK ? count - done : CKPT_CHUNK;
            if (fread(stage.data(), sizeof(float), n, f) != n) return fail(ANE_CUDA_ERR_INVALID, "%s: %s is truncated", __func__, path);
            ANE_CUDA_TRY(cudaMemcpy(dst[which] + off + done, stage.data(), n * sizeof(float), cudaMemcpyHostToDevice));
        }
        return ANE_CUDA_OK;
    });
    fclose(f);
    return rc;
}

static int ckpt_save(Layout layout, const char *path, const ane_ckpt_header *hdr, const float *w_dev, const float *m_dev,
                     const float *v_dev, size_t n_floats) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(path && hdr && w_dev && m_dev && v_dev, "%s: null pointer", __func__);
    ANE_REQUIRE(hdr->magic == CKPT_MAGIC && (hdr->version == 2 || hdr->version == 4), "%s: bad header", __func__);
    ANE_REQUIRE(param_count(*hdr) > 0 && (layout == WEIGHT_ORDER ? param_count(*hdr) == n_floats : param_count(*hdr) <= n_floats),
                "%s: the header describes %zu parameters, the buffers %zu", __func__, param_count(*hdr), n_floats);
    FILE *f = fopen(path, "wb");
    if (!f) return fail(ANE_CUDA_ERR_INVALID, "%s: cannot create %s", __func__, path);
    int rc = fwrite(hdr, sizeof(*hdr), 1, f) == 1 ? ANE_CUDA_OK : fail(ANE_CUDA_ERR_INVALID, "%s: write failed", __func__);
    std::vector<float> stage(CKPT_CHUNK);
    const float *src[3] = {w_dev, m_dev, v_dev};
    if (rc == ANE_CUDA_OK)
        rc = walk(*hdr, layout, [&](int which, size_t off, size_t count) -> int {
            for (size_t done = 0; done < count; done += CKPT_CHUNK) {
                const size_t n = count - done < CKPT_CHUNK ? count - done : CKPT_CHUNK;
                ANE_CUDA_TRY(cudaMemcpy(stage.data(), src[which] + off + done, n * sizeof(float), cudaMemcpyDeviceToHost));
                if (fwrite(stage.data(), sizeof(float), n, f) != n) return fail(ANE_CUDA_ERR_INVALID, "%s: write failed", __func__);
            }
            return ANE_CUDA_OK;
        });
    if (fclose(f) != 0 && rc == ANE_CUDA_OK) rc = fail(ANE_CUDA_ERR_INVALID, "%s: close failed", __func__);
    return rc;
}

int ane_cuda_ckpt_load(const char *path, ane_ckpt_header *hdr, float *w_dev, float *m_dev, float *v_dev, size_t n_floats) {
    return ckpt_load(WEIGHT_ORDER, path, hdr, w_dev, m_dev, v_dev, n_floats);
}
int ane_cuda_ckpt_save(const char *path, const ane_ckpt_header *hdr, const float *w_dev, const float *m_dev, const float *v_dev,
                       size_t n_floats) {
    return ckpt_save(WEIGHT_ORDER, path, hdr, w_dev, m_dev, v_dev, n_floats);
}
int ane_cuda_ckpt_load_flat(const char *path, ane_ckpt_header *hdr, float *w_dev, float *m_dev, float *v_dev, size_t n_floats) {
    return ckpt_load(OPTIMIZER_ORDER, path, hdr, w_dev, m_dev, v_dev, n_floats);
}
int ane_cuda_ckpt_save_flat(const char *path, const ane_ckpt_header *hdr, const float *w_dev, const float *m_dev, const float *v_dev,
                            size_t n_floats) {
    return ckpt_save(OPTIMIZER_ORDER, path, hdr, w_dev, m_dev, v_dev, n_floats);
}

size_t ane_cuda_ckpt_flat_decay_count(const ane_ckpt_header *hdr) {
    if (!hdr || param_count(*hdr) == 0) return 0;
    return tensor_offset(*hdr, OPTIMIZER_ORDER, T_RMS_ATT, 0);
}

int ane_cuda_ckpt_tensor_offset(const ane_ckpt_header *hdr, int flat, int tensor, int layer, size_t *offset, size_t *count) {
    ANE_REQUIRE(hdr && offset && count, "%s: null pointer", __func__);
    ANE_REQUIRE(param_count(*hdr) > 0, "%s: bad header", __func__);
    ANE_REQUIRE(tensor >= 0 && tensor <= T_EMBED && layer >= 0 && layer < hdr->n_layers, "%s: no tensor %d in layer %d", __func__, tensor, layer);
    size_t sz[9];
    layer_extents(*hdr, sz);
    *offset = tensor_offset(*hdr, flat ? OPTIMIZER_ORDER : WEIGHT_ORDER, tensor, tensor < 9 ? layer : 0);
    *count = tensor < 9 ? sz[tensor] : tensor == T_RMS_FINAL ? (size_t)hdr->dim : (size_t)hdr->vocab_size * hdr->dim;
    return ANE_CUDA_OK;
}

// ------------------------------------------------------------------ llama2.c weight files (train_large.m:13-56)
int ane_cuda_llama2c_read_config(const char *path, ane_llama2c_config *cfg) {
    ANE_REQUIRE(path && cfg, "%s: null pointer", __func__);
    FILE *f = fopen(path, "rb");
    if (!f) return fail(ANE_CUDA_ERR_INVALID, "%s: cannot open %s", __func__, path);
    const size_t got = fread(cfg, sizeof(*cfg), 1, f);
    fclose(f);
    if (got != 1) return fail(ANE_CUDA_ERR_INVALID, "%s: %s is shorter than its 28-byte header", __func__, path);
    if (cfg->dim < 1 || cfg->hidden_dim < 1 || cfg->n_layers < 1 || cfg->n_heads < 1 || cfg->n_kv_heads < 1 || cfg->vocab_size == 0 ||
        cfg->dim % cfg->n_heads != 0 || cfg->n_heads % cfg->n_kv_heads != 0)
        return fail(ANE_CUDA_ERR_INVALID, "%s: inconsistent dimensions in the header of %s", __func__, path);
    return ANE_CUDA_OK;
}

int ane_cuda_llama2c_to_header(const ane_llama2c_config *cfg, ane_ckpt_header *hdr) {
    ANE_REQUIRE(cfg && hdr, "%s: null pointer", __func__);
    memset(hdr, 0, sizeof(*hdr));
    const bool gqa = cfg->n_kv_heads != cfg->n_heads;
    hdr->magic = CKPT_MAGIC;
    hdr->version = gqa ? 4 : 2;       // the square-attention files of train_large.m are version 2, grouped-query ones version 4
    hdr->n_layers = cfg->n_layers;
    hdr->vocab_size = cfg->vocab_size < 0 ? -cfg->vocab_size : cfg->vocab_size;      // sign = shared classifier (train_large.m:25-26)
    hdr->dim = cfg->dim;
    hdr->hidden_dim = cfg->hidden_dim;
    hdr->n_heads = cfg->n_heads;
    hdr->seq_len = cfg->seq_len;
    if (gqa) {
        hdr->head_dim = cfg->dim / cfg->n_heads;
        hdr->kv_heads = cfg->n_kv_heads;
        hdr->q_dim = cfg->dim;
    }
    return param_count(*hdr) ? ANE_CUDA_OK : fail(ANE_CUDA_ERR_INVALID, "%s: inconsistent dimensions", __func__);
}

int ane_cuda_llama2c_load(const char *path, const ane_llama2c_config *expect, ane_ckpt_header *hdr, float *w_dev, size_t n_floats, int flat) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(path && hdr && w_dev, "%s: null pointer", __func__);
    ane_llama2c_config cfg;
    if (int rc = ane_cuda_llama2c_read_config(path, &cfg)) return rc;
    if (expect && (cfg.dim != expect->dim || cfg.hidden_dim != expect->hidden_dim || cfg.n_layers != expect->n_layers))
        return fail(ANE_CUDA_ERR_INVALID, "%s: config mismatch: the file has dim=%d hidden=%d layers=%d, expected dim=%d hidden=%d layers=%d",
                    __func__, cfg.dim, cfg.hidden_dim, cfg.n_layers, expect->dim, expect->hidden_dim, expect->n_layers);
    if (int rc = ane_cuda_llama2c_to_header(&cfg, hdr)) return rc;
    const Layout layout = flat ? OPTIMIZER_ORDER : WEIGHT_ORDER;
    if (flat ? param_count(*hdr) > n_floats : param_count(*hdr) != n_floats)
        return fail(ANE_CUDA_ERR_INVALID, "%s: the file holds %zu parameters, the buffer %zu", __func__, param_count(*hdr), n_floats);
    FILE *f = fopen(path, "rb");
    if (!f) return fail(ANE_CUDA_ERR_INVALID, "%s: cannot open %s", __func__, path);
    if (fseek(f, (long)sizeof(cfg), SEEK_SET) != 0) { fclose(f); return fail(ANE_CUDA_ERR_INVALID, "%s: seek failed", __func__); }
    size_t sz[9];
    layer_extents(*hdr, sz);
    std::vector<float> stage(CKPT_CHUNK);
    auto read_to = [&](size_t off, size_t count) -> int {
        for (size_t done = 0; done < count; done += CKPT_CHUNK) {
            const size_t n = count - done < CKPT_CHUNK ? count - done : CKPT_CHUNK;
            if (fread(stage.data(), sizeof(float), n, f) != n) return fail(ANE_CUDA_ERR_INVALID, "%s: %s is truncated", __func__, path);
            ANE_CUDA_TRY(cudaMemcpy(w_dev + off + done, stage.data(), n * sizeof(float), cudaMemcpyHostToDevice));
        }
        return ANE_CUDA_OK;
    };
    // file order: embed, then each kind of tensor for all layers
    static const int order[9] = {T_RMS_ATT, T_WQ, T_WK, T_WV, T_WO, T_RMS_FFN, T_W1, T_W2, T_W3};
    int rc = read_to(tensor_offset(*hdr, layout, T_EMBED, 0), (size_t)hdr->vocab_size * hdr->dim);
    for (int k = 0; k < 9 && rc == ANE_CUDA_OK; k++)
        for (int L = 0; L < hdr->n_layers && rc == ANE_CUDA_OK; L++) rc = read_to(tensor_offset(*hdr, layout, order[k], L), sz[order[k]]);
    if (rc == ANE_CUDA_OK) rc = read_to(tensor_offset(*hdr, layout, T_RMS_FINAL, 0), (size_t)hdr->dim);
    fclose(f);
    return rc;
}

}  // extern "C"
