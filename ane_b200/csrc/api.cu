// api.cu -- lifecycle, device buffers, scratch management and the host-pointer drop-ins of
// libane_cuda.  The boundary is modelled on bridge/ane_bridge.h:16-94 (opaque handles, int
// status, byte-count read/write, explicit free); the drop-ins keep the argument order and
// the overwrite / accumulate behaviour of training/stories_cpu_ops.h and
// training/training_dynamic/cpu_ops.h.
#include "common.cuh"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <math.h>

struct ANECudaBuf {
    void *dev;
    size_t bytes;
};

namespace ane {

static Context g_ctx;
static thread_local char g_err[512] = "";
static std::atomic<long long> g_launches{0};

Context &ctx() { return g_ctx; }

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

void note_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

void *workspace(size_t bytes) {
    Context &c = g_ctx;
    if (bytes <= c.ws_bytes && c.ws) return c.ws;
    // Grow: cudaFree waits for all work on the device, so kernels still using the old range finish first.
    if (c.ws) { cudaFree(c.ws); c.ws = nullptr; c.ws_bytes = 0; }
    const size_t want = round_up(bytes + bytes / 4, (size_t)1 << 20);
    void *p = nullptr;
    if (cudaMalloc(&p, want) != cudaSuccess) {
        cudaGetLastError();
        if (cudaMalloc(&p, round_up(bytes, 256)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        c.ws_bytes = round_up(bytes, 256);
    } else {
        c.ws_bytes = want;
    }
    c.ws = p;
    return p;
}

// Device staging for the host-pointer drop-ins (separate from the kernels' scratch).
struct Stage {
    char *base = nullptr;
    size_t off = 0;
    template <typename P> P *take(size_t bytes) {
        P *p = reinterpret_cast<P *>(base + off);
        off += round_up(bytes, 256);
        return p;
    }
};

static int stage_reserve(Stage &s, size_t total) {
    Context &c = g_ctx;
    total += 4096;
    if (total > c.stage_bytes) {
        if (c.stage) { cudaFree(c.stage); c.stage = nullptr; c.stage_bytes = 0; }
        void *p = nullptr;
        if (cudaMalloc(&p, total) != cudaSuccess) { cudaGetLastError(); return fail(ANE_CUDA_ERR_NOMEM, "staging: cudaMalloc(%zu) failed", total); }
        c.stage = p;
        c.stage_bytes = total;
    }
    s.base = static_cast<char *>(c.stage);
    s.off = 0;
    return ANE_CUDA_OK;
}

static inline size_t pad(size_t b) { return round_up(b, 256); }

}  // namespace ane

using namespace ane;

#define H2D(dst, src, bytes) ANE_CUDA_TRY(cudaMemcpyAsync((dst), (src), (bytes), cudaMemcpyHostToDevice, 0))
#define D2H(dst, src, bytes) ANE_CUDA_TRY(cudaMemcpyAsync((dst), (src), (bytes), cudaMemcpyDeviceToHost, 0))
#define SYNC0() ANE_CUDA_TRY(cudaStreamSynchronize(0))
#define TRY(expr) do { int rc__ = (expr); if (rc__ != ANE_CUDA_OK) return rc__; } while (0)

extern "C" {

int ane_cuda_version(void) { return ANE_CUDA_VERSION; }

const char *ane_cuda_last_error(void) { return g_err; }

long long ane_cuda_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
void ane_cuda_reset_launch_count(void) { g_launches.store(0, std::memory_order_relaxed); }

int ane_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

int ane_cuda_init(int device) {
    Context &c = g_ctx;
    if (c.inited) {
        if (c.device == device) return ANE_CUDA_OK;
        return fail(ANE_CUDA_ERR_INVALID, "ane_cuda_init: already initialised on device %d (one device per process)", c.device);
    }
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        return fail(ANE_CUDA_ERR_CUDA, "ane_cuda_init: no CUDA device (%s); this library has no CPU path", cudaGetErrorString(e));
    }
    ANE_REQUIRE(device >= 0 && device < n, "ane_cuda_init: device %d out of range [0,%d)", device, n);
    ANE_CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    ANE_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return fail(ANE_CUDA_ERR_UNSUPPORTED, "ane_cuda_init: device %d is sm_%d%d; the kernels are built for sm_100a only", device, prop.major, prop.minor);
    c.sm_count = prop.multiProcessorCount;
    ANE_CUDA_TRY(cudaMalloc(reinterpret_cast<void **>(&c.status), sizeof(ane_cuda_status)));
    ANE_CUDA_TRY(cudaMemset(c.status, 0, sizeof(ane_cuda_status)));
    c.device = device;
    c.inited = true;
    return ANE_CUDA_OK;
}

void ane_cuda_shutdown(void) {
    Context &c = g_ctx;
    if (!c.inited) return;
    cudaDeviceSynchronize();
    if (c.ws) cudaFree(c.ws);
    if (c.stage) cudaFree(c.stage);
    if (c.status) cudaFree(c.status);
    if (c.pinned) cudaFreeHost(c.pinned);
    c = Context();
}

ANECudaBuf *ane_cuda_alloc(size_t bytes) {
    if (!g_ctx.inited) { fail(ANE_CUDA_ERR_NOT_INIT, "ane_cuda_alloc: call ane_cuda_init first"); return nullptr; }
    if (bytes == 0) { fail(ANE_CUDA_ERR_INVALID, "ane_cuda_alloc: zero bytes"); return nullptr; }
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); fail(ANE_CUDA_ERR_NOMEM, "ane_cuda_alloc: cudaMalloc(%zu) failed", bytes); return nullptr; }
    ANECudaBuf *b = new ANECudaBuf{p, bytes};
    return b;
}

int ane_cuda_write(ANECudaBuf *buf, size_t offset, const void *host, size_t bytes) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(buf && host, "%s: null pointer", __func__);
    ANE_REQUIRE(offset <= buf->bytes && bytes <= buf->bytes - offset, "%s: range [%zu, %zu) outside buffer of %zu bytes", __func__, offset, offset + bytes, buf->bytes);
    ANE_CUDA_TRY(cudaMemcpy(static_cast<char *>(buf->dev) + offset, host, bytes, cudaMemcpyHostToDevice));
    return ANE_CUDA_OK;
}

int ane_cuda_read(ANECudaBuf *buf, size_t offset, void *host, size_t bytes) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(buf && host, "%s: null pointer", __func__);
    ANE_REQUIRE(offset <= buf->bytes && bytes <= buf->bytes - offset, "%s: range [%zu, %zu) outside buffer of %zu bytes", __func__, offset, offset + bytes, buf->bytes);
    ANE_CUDA_TRY(cudaMemcpy(host, static_cast<char *>(buf->dev) + offset, bytes, cudaMemcpyDeviceToHost));
    return ANE_CUDA_OK;
}

void *ane_cuda_devptr(ANECudaBuf *buf) { return buf ? buf->dev : nullptr; }
size_t ane_cuda_bufsize(ANECudaBuf *buf) { return buf ? buf->bytes : 0; }

void ane_cuda_free(ANECudaBuf *buf) {
    if (!buf) return;
    if (buf->dev) cudaFree(buf->dev);
    delete buf;
}

void *ane_cuda_host_alloc(size_t bytes) {
    if (!g_ctx.inited) { fail(ANE_CUDA_ERR_NOT_INIT, "ane_cuda_host_alloc: call ane_cuda_init first"); return nullptr; }
    void *p = nullptr;
    if (cudaMallocHost(&p, bytes) != cudaSuccess) { cudaGetLastError(); fail(ANE_CUDA_ERR_NOMEM, "ane_cuda_host_alloc: cudaMallocHost(%zu) failed", bytes); return nullptr; }
    return p;
}

void ane_cuda_host_free(void *p) { if (p) cudaFreeHost(p); }

int ane_cuda_sync(void *stream) {
    ANE_REQUIRE_INIT();
    ANE_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    return ANE_CUDA_OK;
}

int ane_cuda_poll_status(ane_cuda_status *out, int reset) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out, "%s: null pointer", __func__);
    ANE_CUDA_TRY(cudaDeviceSynchronize());
    ANE_CUDA_TRY(cudaMemcpy(out, g_ctx.status, sizeof(*out), cudaMemcpyDeviceToHost));
    if (reset) ANE_CUDA_TRY(cudaMemset(g_ctx.status, 0, sizeof(ane_cuda_status)));
    return ANE_CUDA_OK;
}

size_t ane_cuda_workspace_bytes(void) { return g_ctx.ws_bytes; }

// ===================================================================== host-pointer drop-ins
int ane_cuda_rmsnorm(float *out, const float *x, const float *w, int d, int S) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && x && w && d > 0 && S > 0, "%s: bad argument", __func__);
    const size_t nb = (size_t)d * S * 4;
    Stage s;
    TRY(stage_reserve(s, 2 * pad(nb) + pad((size_t)d * 4)));
    float *dx_ = s.take<float>(nb), *dout = s.take<float>(nb), *dw_ = s.take<float>((size_t)d * 4);
    H2D(dx_, x, nb);
    H2D(dw_, w, (size_t)d * 4);
    TRY(ane_cuda_rmsnorm_dev(0, ANE_F32, 1, d, S, dout, dx_, dw_, 1e-5f));   // eps literal of stories_cpu_ops.h:13
    D2H(out, dout, nb);
    SYNC0();
    return ANE_CUDA_OK;
}

int ane_cuda_rmsnorm_bwd(float *dx, float *dw, const float *dy, const float *x, const float *w, int d, int S) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dx && dw && dy && x && w && d > 0 && S > 0, "%s: bad argument", __func__);
    const size_t nb = (size_t)d * S * 4, wb = (size_t)d * 4;
    Stage s;
    TRY(stage_reserve(s, 3 * pad(nb) + 2 * pad(wb)));
    float *ddx = s.take<float>(nb), *ddy = s.take<float>(nb), *dx_ = s.take<float>(nb);
    float *dw_ = s.take<float>(wb), *ddw = s.take<float>(wb);
    H2D(ddy, dy, nb);
    H2D(dx_, x, nb);
    H2D(dw_, w, wb);
    H2D(ddw, dw, wb);                                                           // dw is accumulated into (:50)
    TRY(ane_cuda_rmsnorm_bwd_dev(0, ANE_F32, 1, d, S, ddx, ddw, ddy, dx_, dw_, nullptr, 1e-5f, ANE_NORM_BWD_REFERENCE));
    D2H(dx, ddx, nb);
    D2H(dw, ddw, wb);
    SYNC0();
    return ANE_CUDA_OK;
}

static int adam_host(float *w, const float *g, AdamState *st, int t, float lr, float b1, float b2, float eps, float wd, unsigned variant) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(w && g && st && st->m && st->v, "adam_update: null pointer");
    const size_t n = st->n, nb = n * 4;
    if (n == 0) return ANE_CUDA_OK;
    Stage s;
    TRY(stage_reserve(s, 4 * pad(nb)));
    float *dw_ = s.take<float>(nb), *dg = s.take<float>(nb), *dm = s.take<float>(nb), *dv = s.take<float>(nb);
    H2D(dw_, w, nb);
    H2D(dg, g, nb);
    H2D(dm, st->m, nb);
    H2D(dv, st->v, nb);
    TRY(ane_cuda_adam_dev(0, n, dw_, dg, dm, dv, t, lr, b1, b2, eps, wd, 1.0f, nullptr, variant));
    D2H(w, dw_, nb);
    D2H(st->m, dm, nb);
    D2H(st->v, dv, nb);
    SYNC0();
    return ANE_CUDA_OK;
}

int ane_cuda_adam_update(float *w, const float *g, AdamState *s, int t, float lr, float b1, float b2, float eps) {
    return adam_host(w, g, s, t, lr, b1, b2, eps, 0.0f, ANE_ADAM_STORIES);
}

int ane_cuda_adam_update_wd(float *w, const float *g, AdamState *s, int t, float lr, float b1, float b2, float eps, float wd) {
    return adam_host(w, g, s, t, lr, b1, b2, eps, wd, ANE_ADAM_DYNAMIC);
}

int ane_cuda_cross_entropy_loss(float *loss, float *dlogits, const float *logits, const uint16_t *targets, int V, int S) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(loss && dlogits && logits && targets && V > 0 && S > 0, "%s: bad argument", __func__);
    const size_t nb = (size_t)V * S * 4;
    Stage s;
    TRY(stage_reserve(s, pad(nb) + pad((size_t)S * 2) + 256));
    float *dl = s.take<float>(nb);
    uint16_t *dt = s.take<uint16_t>((size_t)S * 2);
    float *dloss = s.take<float>(4);
    H2D(dl, logits, nb);
    H2D(dt, targets, (size_t)S * 2);
    TRY(ane_cuda_cross_entropy_dev(0, ANE_ID_U16, 1, V, S, dl, dl, dt, dloss, 1.0f));   // in place on the device
    D2H(dlogits, dl, nb);
    D2H(loss, dloss, 4);
    SYNC0();
    return ANE_CUDA_OK;
}

int ane_cuda_embed_lookup(float *x, const float *embed, const uint16_t *tokens, int dim, int seq, int vocab) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(x && embed && tokens && dim > 0 && seq > 0 && vocab > 0, "%s: bad argument", __func__);
    const size_t xb = (size_t)dim * seq * 4, eb = (size_t)vocab * dim * 4;
    Stage s;
    TRY(stage_reserve(s, pad(xb) + pad(eb) + pad((size_t)seq * 2)));
    float *dx_ = s.take<float>(xb), *de = s.take<float>(eb);
    uint16_t *dt = s.take<uint16_t>((size_t)seq * 2);
    H2D(dx_, x, xb);                      // columns of out-of-range ids keep the caller's values (:115)
    H2D(de, embed, eb);
    H2D(dt, tokens, (size_t)seq * 2);
    TRY(ane_cuda_embed_lookup_dev(0, ANE_F32, ANE_ID_U16, 1, dim, seq, dx_, de, dt, vocab, ANE_OOR_SKIP));
    D2H(x, dx_, xb);
    SYNC0();
    return ANE_CUDA_OK;
}

int ane_cuda_embed_backward(float *d_embed, const float *dx, const uint16_t *tokens, int dim, int seq, int vocab) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(d_embed && dx && tokens && dim > 0 && seq > 0 && vocab > 0, "%s: bad argument", __func__);
    const size_t xb = (size_t)dim * seq * 4, eb = (size_t)vocab * dim * 4;
    Stage s;
    TRY(stage_reserve(s, pad(xb) + pad(eb) + pad((size_t)seq * 2)));
    float *dx_ = s.take<float>(xb), *de = s.take<float>(eb);
    uint16_t *dt = s.take<uint16_t>((size_t)seq * 2);
    H2D(dx_, dx, xb);
    H2D(de, d_embed, eb);
    H2D(dt, tokens, (size_t)seq * 2);
    TRY(ane_cuda_embed_backward_dev(0, ANE_F32, ANE_ID_U16, 1, dim, seq, de, dx_, dt, vocab));
    D2H(d_embed, de, eb);
    SYNC0();
    return ANE_CUDA_OK;
}

int ane_cuda_rope_backward_inplace(float *dx, int seq, int dim, int hd) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dx && seq > 0 && dim > 0 && hd > 0, "%s: bad argument", __func__);
    const size_t nb = (size_t)dim * seq * 4;
    Stage s;
    TRY(stage_reserve(s, pad(nb)));
    float *d = s.take<float>(nb);
    H2D(d, dx, nb);
    TRY(ane_cuda_rope_dev(0, ANE_F32, 1, dim, seq, hd, d, d, 10000.0f, 0, ANE_ROPE_INVERSE));   // base literal of cpu_ops.h:172
    D2H(dx, d, nb);
    SYNC0();
    return ANE_CUDA_OK;
}

int ane_cuda_residual(float *out, const float *x, const float *f, float alpha, size_t n) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && x && f, "%s: null pointer", __func__);
    if (n == 0) return ANE_CUDA_OK;
    Stage s;
    TRY(stage_reserve(s, 2 * pad(n * 4)));
    float *a = s.take<float>(n * 4), *b = s.take<float>(n * 4);
    H2D(a, x, n * 4);
    H2D(b, f, n * 4);
    TRY(ane_cuda_residual_dev(0, ANE_F32, n, a, a, b, alpha));
    D2H(out, a, n * 4);
    SYNC0();
    return ANE_CUDA_OK;
}

int ane_cuda_swiglu(float *out, const float *h1, const float *h3, size_t n) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && h1 && h3, "%s: null pointer", __func__);
    if (n == 0) return ANE_CUDA_OK;
    Stage s;
    TRY(stage_reserve(s, 2 * pad(n * 4)));
    float *a = s.take<float>(n * 4), *b = s.take<float>(n * 4);
    H2D(a, h1, n * 4);
    H2D(b, h3, n * 4);
    TRY(ane_cuda_swiglu_dev(0, ANE_F32, n, a, a, b));
    D2H(out, a, n * 4);
    SYNC0();
    return ANE_CUDA_OK;
}

int ane_cuda_swiglu_bwd(float *dh1, float *dh3, const float *h1, const float *h3, const float *dsilu, size_t n) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dh1 && dh3 && h1 && h3 && dsilu, "%s: null pointer", __func__);
    if (n == 0) return ANE_CUDA_OK;
    Stage s;
    TRY(stage_reserve(s, 3 * pad(n * 4)));
    float *a = s.take<float>(n * 4), *b = s.take<float>(n * 4), *c = s.take<float>(n * 4);
    H2D(a, h1, n * 4);
    H2D(b, h3, n * 4);
    H2D(c, dsilu, n * 4);
    TRY(ane_cuda_swiglu_bwd_dev(0, ANE_F32, n, a, b, a, b, c));   // dh1 over h1, dh3 over h3
    D2H(dh1, a, n * 4);
    D2H(dh3, b, n * 4);
    SYNC0();
    return ANE_CUDA_OK;
}

}  // extern "C"
