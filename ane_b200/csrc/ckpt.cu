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

// One pass over the file's tensors in file order.  io(dev_buffer_index 0/1/2 = w/m/v, offset in floats, count) moves
// `count` floats between the file position and the device range.
template <class IO>
static int walk(const ane_ckpt_header &h, IO io) {
    size_t sz[9];
    layer_extents(h, sz);
    size_t off = 0;
    for (int L = 0; L < h.n_layers; L++) {
        size_t o = off;
        for (int i = 0; i < 9; i++) { if (int rc = io(0, o, sz[i])) return rc; o += sz[i]; }
        o = off;
        for (int i = 0; i < 9; i++) {
            if (int rc = io(1, o, sz[i])) return rc;
            if (int rc = io(2, o, sz[i])) return rc;
            o += sz[i];
        }
        off = o;
    }
    const size_t d = (size_t)h.dim, e = (size_t)h.vocab_size * h.dim;
    if (int rc = io(0, off, d)) return rc;
    if (int rc = io(1, off, d)) return rc;
    if (int rc = io(2, off, d)) return rc;
    off += d;
    if (int rc = io(0, off, e)) return rc;
    if (int rc = io(1, off, e)) return rc;
    if (int rc = io(2, off, e)) return rc;
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

int ane_cuda_ckpt_load(const char *path, ane_ckpt_header *hdr, float *w_dev, float *m_dev, float *v_dev, size_t n_floats) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(path && hdr && w_dev, "%s: null pointer", __func__);
    ANE_REQUIRE((m_dev == nullptr) == (v_dev == nullptr), "%s: give both moment buffers or neither", __func__);
    FILE *f = fopen(path, "rb");
    if (!f) return fail(ANE_CUDA_ERR_INVALID, "%s: cannot open %s", __func__, path);
    int rc = read_header(f, hdr);
    if (rc == ANE_CUDA_OK && param_count(*hdr) != n_floats)
        rc = fail(ANE_CUDA_ERR_INVALID, "%s: the file holds %zu parameters, the buffers %zu", __func__, param_count(*hdr), n_floats);
    if (rc != ANE_CUDA_OK) { fclose(f); return rc; }
    std::vector<float> stage(CKPT_CHUNK);
    float *dst[3] = {w_dev, m_dev, v_dev};
    rc = walk(*hdr, [&](int which, size_t off, size_t count) -> int {
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

int ane_cuda_ckpt_save(const char *path, const ane_ckpt_header *hdr, const float *w_dev, const float *m_dev, const float *v_dev,
                       size_t n_floats) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(path && hdr && w_dev && m_dev && v_dev, "%s: null pointer", __func__);
    ANE_REQUIRE(hdr->magic == CKPT_MAGIC && (hdr->version == 2 || hdr->version == 4), "%s: bad header", __func__);
    ANE_REQUIRE(param_count(*hdr) == n_floats && n_floats > 0, "%s: the header describes %zu parameters, the buffers %zu", __func__,
                param_count(*hdr), n_floats);
    FILE *f = fopen(path, "wb");
    if (!f) return fail(ANE_CUDA_ERR_INVALID, "%s: cannot create %s", __func__, path);
    int rc = fwrite(hdr, sizeof(*hdr), 1, f) == 1 ? ANE_CUDA_OK : fail(ANE_CUDA_ERR_INVALID, "%s: write failed", __func__);
    std::vector<float> stage(CKPT_CHUNK);
    const float *src[3] = {w_dev, m_dev, v_dev};
    if (rc == ANE_CUDA_OK)
        rc = walk(*hdr, [&](int which, size_t off, size_t count) -> int {
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

}  // extern "C"
