// api.cu -- lifecycle, device buffers, scratch management and the host-pointer drop-ins of
// libane_cuda.  The boundary is modelled on bridge/ane_bridge.h:16-94 (opaque handles, int
// status, byte-count read/write, explicit free); the drop-ins keep the argument order and
// the overwrite / accumulate behaviour of training/stories_cpu_ops.h and
// training/training_dynamic/cpu_ops.h.
#include "common.cuh"

#include <vector>
#include "tma.cuh"

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

// cuTensorMapEncodeTiled is a driver entry point; it is resolved through the runtime so that the
// library does not link against libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode_tiled = nullptr;

int make_bcs_tensor_map(CUtensorMap *map, ane_dtype dtype, const void *base, int B, int C, int S, int box_s, int box_c,
                        int l2_promotion_bytes) {
    if (!g_encode_tiled) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return fail(ANE_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        }
        g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    }
    const size_t e = dtype_size(dtype);
    if (!aligned16(base) || ((size_t)S * e) % 16 || ((size_t)box_s * e) % 16 || box_s > 256 || box_c > 256 || box_s < 1 || box_c < 1)
        return fail(ANE_CUDA_ERR_INVALID, "tensor map: unsupported alignment or box (S=%d box %dx%d)", S, box_s, box_c);
    const CUtensorMapDataType dt = dtype == ANE_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == ANE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const cuuint64_t dims[3] = {(cuuint64_t)S, (cuuint64_t)C, (cuuint64_t)B};
    const cuuint64_t strides[2] = {(cuuint64_t)S * e, (cuuint64_t)C * S * e};
    const cuuint32_t box[3] = {(cuuint32_t)box_s, (cuuint32_t)box_c, 1u};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    const CUtensorMapL2promotion promo = l2_promotion_bytes >= 256 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B
                                       : l2_promotion_bytes >= 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                       : l2_promotion_bytes >= 64 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B : CU_TENSOR_MAP_L2_PROMOTION_NONE;
    const CUresult r = g_encode_tiled(map, dt, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                      CU_TENSOR_MAP_SWIZZLE_NONE, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ANE_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return ANE_CUDA_OK;
}

struct Knob { char name[32]; int value; };
static Knob g_knobs[32];
static int g_nknobs = 0;

int tuning(const char *name, int dflt) {
    for (int i = 0; i < g_nknobs; i++)
        if (strcmp(g_knobs[i].name, name) == 0) return g_knobs[i].value;
    return dflt;
}

bool check_extents_on() { return tuning("check_extents", 0) != 0; }

int check_extent(const char *fn, const char *what, const void *p, size_t bytes) {
    typedef CUresult (*RangeFn)(CUdeviceptr *, size_t *, CUdeviceptr);
    static RangeFn range = nullptr;
    if (!range) {
        cudaDriverEntryPointQueryResult qr;
        void *f = nullptr;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &qr) != cudaSuccess || !f) {
            cudaGetLastError();
            return ANE_CUDA_OK;          // cannot check on this driver: do not block the call
        }
        range = reinterpret_cast<RangeFn>(f);
    }
    CUdeviceptr base = 0;
    size_t size = 0;
    if (range(&base, &size, (CUdeviceptr)p) != CUDA_SUCCESS)
        return fail(ANE_CUDA_ERR_INVALID, "%s: %s = %p is not inside a device allocation", fn, what, p);
    const size_t off = (size_t)((CUdeviceptr)p - base);
    if (bytes > size - off)
        return fail(ANE_CUDA_ERR_INVALID, "%s: %s needs %zu bytes but its allocation has only %zu left from that address", fn, what, bytes, size - off);
    return ANE_CUDA_OK;
}

static std::vector<void *> g_retired;      // device ranges replaced by larger ones; freed at shutdown
static bool g_frozen = false;

bool frozen() { return g_frozen; }
void retire_device_range(void *p) { if (p) g_retired.push_back(p); }

cudaError_t dev_malloc(void **p, size_t bytes) {
    for (int i = 0; i < g_nknobs; i++)
        if (strcmp(g_knobs[i].name, "fail_alloc") == 0 && g_knobs[i].value > 0) {
            g_knobs[i].value--;
            *p = nullptr;
            return cudaErrorMemoryAllocation;
        }
    const cudaError_t e = cudaMalloc(p, bytes);
    if (e != cudaSuccess) cudaGetLastError();
    return e;
}

void *workspace(size_t bytes) {
    Context &c = g_ctx;
    if (bytes <= c.ws_bytes && c.ws) return c.ws;
    if (g_frozen) return nullptr;       // the caller reports "no scratch"; ane_cuda_reserve_workspace before freezing avoids it
    // Grow into a NEW range.  The old one stays allocated until shutdown: kernels already enqueued and CUDA graphs already
    // captured keep a valid address (each launch fully rewrites the part of the scratch it reads, so an old and a new
    // range never have to agree).
    const size_t want = round_up(bytes + bytes / 4, (size_t)1 << 20);
    void *p = nullptr;
    size_t got = want;
    if (dev_malloc(&p, want) != cudaSuccess) {
        got = round_up(bytes, 256);
        if (dev_malloc(&p, got) != cudaSuccess) return nullptr;
    }
    retire_device_range(c.ws);
    c.ws = p;
    c.ws_bytes = got;
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
        if (c.stage) { cudaFree(c.stage); c.stage = nullptr; c.stage_bytes = 0; }      // host-buffer calls are synchronous: nothing refers to it
        void *p = nullptr;
        if (dev_malloc(&p, total) != cudaSuccess) return fail(ANE_CUDA_ERR_NOMEM, "staging: cudaMalloc(%zu) failed", total);
        c.stage = p;
        c.stage_bytes = total;
    }
    s.base = static_cast<char *>(c.stage);
    s.off = 0;
    return ANE_CUDA_OK;
}

static inline size_t pad(size_t b) { return round_up(b, 256); }
static void pipe_destroy();

}  // namespace ane

using namespace ane;

#define H2D(dst, src, bytes) ANE_CUDA_TRY(cudaMemcpyAsync((dst), (src), (bytes), cudaMemcpyHostToDevice, 0))
#define D2H(dst, src, bytes) ANE_CUDA_TRY(cudaMemcpyAsync((dst), (src), (bytes), cudaMemcpyDeviceToHost, 0))
#define SYNC0() ANE_CUDA_TRY(cudaStreamSynchronize(0))
#define TRY(expr) do { int rc__ = (expr); if (rc__ != ANE_CUDA_OK) return rc__; } while (0)

extern "C" {

int ane_cuda_version(void) { return ANE_CUDA_VERSION; }

int ane_cuda_set_tuning(const char *name, int value) {
    if (!name || strlen(name) >= sizeof(g_knobs[0].name)) return fail(ANE_CUDA_ERR_INVALID, "ane_cuda_set_tuning: bad knob name");
    for (int i = 0; i < g_nknobs; i++)
        if (strcmp(g_knobs[i].name, name) == 0) { g_knobs[i].value = value; return ANE_CUDA_OK; }
    if (g_nknobs >= 32) return fail(ANE_CUDA_ERR_INVALID, "ane_cuda_set_tuning: too many knobs");
    strcpy(g_knobs[g_nknobs].name, name);
    g_knobs[g_nknobs++].value = value;
    return ANE_CUDA_OK;
}

int ane_cuda_clear_tuning(const char *name) {
    if (!name) { g_nknobs = 0; return ANE_CUDA_OK; }
    for (int i = 0; i < g_nknobs; i++)
        if (strcmp(g_knobs[i].name, name) == 0) {
            g_knobs[i] = g_knobs[g_nknobs - 1];
            g_nknobs--;
            break;
        }
    return ANE_CUDA_OK;
}

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
    ane_cuda_comm_destroy();
    pipe_destroy();
    rope_tables_release();
    embed_side_release();
    qk_side_release();
    if (c.ws) cudaFree(c.ws);
    for (void *p : g_retired) cudaFree(p);
    g_retired.clear();
    g_frozen = false;
    if (c.stage) cudaFree(c.stage);
    if (c.status) cudaFree(c.status);
    if (c.pinned) cudaFreeHost(c.pinned);
    c = Context();
}

ANECudaBuf *ane_cuda_alloc(size_t bytes) {
    if (!g_ctx.inited) { fail(ANE_CUDA_ERR_NOT_INIT, "ane_cuda_alloc: call ane_cuda_init first"); return nullptr; }
    if (bytes == 0) { fail(ANE_CUDA_ERR_INVALID, "ane_cuda_alloc: zero bytes"); return nullptr; }
    void *p = nullptr;
    if (dev_malloc(&p, bytes) != cudaSuccess) { fail(ANE_CUDA_ERR_NOMEM, "ane_cuda_alloc: cudaMalloc(%zu) failed", bytes); return nullptr; }
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

int ane_cuda_zero_dev(void *stream, void *dev, size_t bytes) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dev || bytes == 0, "%s: null pointer", __func__);
    if (bytes) ANE_CUDA_TRY(cudaMemsetAsync(dev, 0, bytes, (cudaStream_t)stream));
    return ANE_CUDA_OK;
}

int ane_cuda_copy_dev(void *stream, void *dst, const void *src, size_t bytes) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE((dst && src) || bytes == 0, "%s: null pointer", __func__);
    if (bytes) ANE_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, (cudaStream_t)stream));
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

int ane_cuda_reserve_workspace(size_t bytes) {
    ANE_REQUIRE_INIT();
    if (bytes == 0) return ANE_CUDA_OK;
    if (!workspace(bytes))
        return fail(g_frozen ? ANE_CUDA_ERR_UNSUPPORTED : ANE_CUDA_ERR_NOMEM, "%s: cannot provide %zu bytes of scratch%s", __func__, bytes,
                    g_frozen ? " (the library is frozen)" : "");
    return ANE_CUDA_OK;
}

int ane_cuda_freeze(int on) {
    ANE_REQUIRE_INIT();
    g_frozen = on != 0;
    return ANE_CUDA_OK;
}

int ane_cuda_release_caches(void) {
    ANE_REQUIRE_INIT();
    ANE_CUDA_TRY(cudaDeviceSynchronize());
    rope_tables_release();
    for (void *p : g_retired) cudaFree(p);
    g_retired.clear();
    return ANE_CUDA_OK;
}

}  // extern "C"

// ===================================================================== host-buffer entry points
// Generic form: activations of any supported dtype in HOST memory, batched [B][C][S].  The batch
// is cut into chunks that flow through a three-stream pipeline (host->device copy, kernel,
// device->host copy) over two staging slots, so PCIe traffic in both directions overlaps the
// kernels.  Page-locked host memory (ane_cuda_host_alloc) makes the copies truly asynchronous;
// pageable memory works but serialises them.
namespace ane {

struct Pipe {
    bool ready = false;
    cudaStream_t s_in = nullptr, s_k = nullptr, s_out = nullptr;
    cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_k[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
};
static Pipe g_pipe;

static int pipe_init() {
    Pipe &p = g_pipe;
    if (p.ready) return ANE_CUDA_OK;
    ANE_CUDA_TRY(cudaStreamCreateWithFlags(&p.s_in, cudaStreamNonBlocking));
    ANE_CUDA_TRY(cudaStreamCreateWithFlags(&p.s_k, cudaStreamNonBlocking));
    ANE_CUDA_TRY(cudaStreamCreateWithFlags(&p.s_out, cudaStreamNonBlocking));
    for (int i = 0; i < 2; i++) {
        ANE_CUDA_TRY(cudaEventCreateWithFlags(&p.ev_in[i], cudaEventDisableTiming));
        ANE_CUDA_TRY(cudaEventCreateWithFlags(&p.ev_k[i], cudaEventDisableTiming));
        ANE_CUDA_TRY(cudaEventCreateWithFlags(&p.ev_out[i], cudaEventDisableTiming));
    }
    p.ready = true;
    return ANE_CUDA_OK;
}

static void pipe_destroy() {
    Pipe &p = g_pipe;
    if (!p.ready) return;
    cudaStreamDestroy(p.s_in); cudaStreamDestroy(p.s_k); cudaStreamDestroy(p.s_out);
    for (int i = 0; i < 2; i++) { cudaEventDestroy(p.ev_in[i]); cudaEventDestroy(p.ev_k[i]); cudaEventDestroy(p.ev_out[i]); }
    p = Pipe();
}

constexpr int MAX_T = 4;
struct HostTensors {
    int n_in = 0, n_out = 0;
    const void *in[MAX_T] = {};
    size_t in_item[MAX_T] = {};     // bytes per item
    void *out[MAX_T] = {};
    size_t out_item[MAX_T] = {};
};

// launch(stream, n_items, dev_in[], dev_out[]) enqueues the kernel(s) for one chunk.
template <class Launch>
static int run_pipelined(size_t items, const HostTensors &ht, size_t extra_stage_bytes, char **extra_stage, Launch launch) {
    TRY(pipe_init());
    Pipe &p = g_pipe;
    size_t per_item = 0;
    for (int i = 0; i < ht.n_in; i++) per_item += ht.in_item[i];
    for (int i = 0; i < ht.n_out; i++) per_item += ht.out_item[i];
    // chunks of about 16 MiB of traffic, at least one item
    size_t chunk = per_item ? ((size_t)16 << 20) / per_item : items;
    if (chunk < 1) chunk = 1;
    if (chunk > items) chunk = items;
    size_t slot_bytes = 0;
    for (int i = 0; i < ht.n_in; i++) slot_bytes += pad(ht.in_item[i] * chunk);
    for (int i = 0; i < ht.n_out; i++) slot_bytes += pad(ht.out_item[i] * chunk);
    Stage st;
    TRY(stage_reserve(st, 2 * slot_bytes + pad(extra_stage_bytes)));
    char *din[2][MAX_T], *dout[2][MAX_T];
    for (int s = 0; s < 2; s++) {
        for (int i = 0; i < ht.n_in; i++) din[s][i] = st.take<char>(ht.in_item[i] * chunk);
        for (int i = 0; i < ht.n_out; i++) dout[s][i] = st.take<char>(ht.out_item[i] * chunk);
    }
    if (extra_stage) *extra_stage = st.take<char>(extra_stage_bytes);
    // work queued earlier on the default stream (e.g. weight uploads by the caller of this helper) is ordered first
    ANE_CUDA_TRY(cudaStreamSynchronize(0));
    size_t done = 0;
    for (size_t c = 0; done < items; c++) {
        const int s = (int)(c & 1);
        const size_t n = items - done < chunk ? items - done : chunk;
        if (c >= 2) ANE_CUDA_TRY(cudaStreamWaitEvent(p.s_in, p.ev_k[s], 0));       // slot inputs consumed
        for (int i = 0; i < ht.n_in; i++)
            ANE_CUDA_TRY(cudaMemcpyAsync(din[s][i], static_cast<const char *>(ht.in[i]) + done * ht.in_item[i], n * ht.in_item[i],
                                         cudaMemcpyHostToDevice, p.s_in));
        ANE_CUDA_TRY(cudaEventRecord(p.ev_in[s], p.s_in));
        ANE_CUDA_TRY(cudaStreamWaitEvent(p.s_k, p.ev_in[s], 0));
        if (c >= 2) ANE_CUDA_TRY(cudaStreamWaitEvent(p.s_k, p.ev_out[s], 0));      // slot outputs drained
        void *vin[MAX_T], *vout[MAX_T];
        for (int i = 0; i < ht.n_in; i++) vin[i] = din[s][i];
        for (int i = 0; i < ht.n_out; i++) vout[i] = dout[s][i];
        TRY(launch(p.s_k, n, vin, vout));
        ANE_CUDA_TRY(cudaEventRecord(p.ev_k[s], p.s_k));
        ANE_CUDA_TRY(cudaStreamWaitEvent(p.s_out, p.ev_k[s], 0));
        for (int i = 0; i < ht.n_out; i++)
            ANE_CUDA_TRY(cudaMemcpyAsync(static_cast<char *>(ht.out[i]) + done * ht.out_item[i], dout[s][i], n * ht.out_item[i],
                                         cudaMemcpyDeviceToHost, p.s_out));
        ANE_CUDA_TRY(cudaEventRecord(p.ev_out[s], p.s_out));
        done += n;
    }
    ANE_CUDA_TRY(cudaStreamSynchronize(p.s_k));
    ANE_CUDA_TRY(cudaStreamSynchronize(p.s_out));
    return ANE_CUDA_OK;
}

static int check_host_shape(const char *fn, ane_dtype dtype, long long B, long long C, long long S) {
    if (!dtype_ok(dtype)) return fail(ANE_CUDA_ERR_INVALID, "%s: bad dtype %d", fn, (int)dtype);
    if (B < 1 || C < 1 || S < 1) return fail(ANE_CUDA_ERR_INVALID, "%s: B, C, S must be positive", fn);
    return ANE_CUDA_OK;
}

}  // namespace ane

extern "C" {

int ane_cuda_rmsnorm_host(ane_dtype dtype, int B, int C, int S, void *out, const void *x, const float *w, float eps) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && x && w, "%s: null pointer", __func__);
    TRY(check_host_shape(__func__, dtype, B, C, S));
    const size_t item = (size_t)C * S * dtype_size(dtype);
    HostTensors ht;
    ht.n_in = 1; ht.in[0] = x; ht.in_item[0] = item;
    ht.n_out = 1; ht.out[0] = out; ht.out_item[0] = item;
    char *ex = nullptr;
    // the weight upload happens inside the first launch closure's stream order
    bool first = true;
    return run_pipelined((size_t)B, ht, (size_t)C * 4, &ex, [&](cudaStream_t st, size_t n, void **di, void **dout_) -> int {
        if (first) { ANE_CUDA_TRY(cudaMemcpyAsync(ex, w, (size_t)C * 4, cudaMemcpyHostToDevice, st)); first = false; }
        return ane_cuda_rmsnorm_dev(st, dtype, (int)n, C, S, dout_[0], di[0], reinterpret_cast<float *>(ex), eps);
    });
}

int ane_cuda_rmsnorm_bwd_host(ane_dtype dtype, int B, int C, int S, void *dx, float *dw, const void *dy, const void *x,
                              const float *w, const void *add, float eps, unsigned flags) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dx && dw && dy && x && w, "%s: null pointer", __func__);
    TRY(check_host_shape(__func__, dtype, B, C, S));
    const size_t item = (size_t)C * S * dtype_size(dtype);
    HostTensors ht;
    ht.n_in = add ? 3 : 2;
    ht.in[0] = dy; ht.in[1] = x; ht.in[2] = add;
    ht.in_item[0] = ht.in_item[1] = ht.in_item[2] = item;
    ht.n_out = 1; ht.out[0] = dx; ht.out_item[0] = item;
    char *ex = nullptr;
    bool first = true;
    const size_t wb = pad((size_t)C * 4);
    cudaStream_t kst = nullptr;
    int rc = run_pipelined((size_t)B, ht, 2 * wb, &ex, [&](cudaStream_t st, size_t n, void **di, void **dout_) -> int {
        float *dw_w = reinterpret_cast<float *>(ex), *dw_dw = reinterpret_cast<float *>(ex + wb);
        if (first) {
            ANE_CUDA_TRY(cudaMemcpyAsync(dw_w, w, (size_t)C * 4, cudaMemcpyHostToDevice, st));
            ANE_CUDA_TRY(cudaMemcpyAsync(dw_dw, dw, (size_t)C * 4, cudaMemcpyHostToDevice, st));   // accumulated into
            first = false;
            kst = st;
        }
        return ane_cuda_rmsnorm_bwd_dev(st, dtype, (int)n, C, S, dout_[0], dw_dw, di[0], di[1], dw_w, add ? di[2] : nullptr, eps, flags);
    });
    if (rc != ANE_CUDA_OK) return rc;
    ANE_CUDA_TRY(cudaMemcpyAsync(dw, ex + wb, (size_t)C * 4, cudaMemcpyDeviceToHost, kst));
    ANE_CUDA_TRY(cudaStreamSynchronize(kst));
    return ANE_CUDA_OK;
}

int ane_cuda_residual_rmsnorm_host(ane_dtype dtype, int B, int C, int S, void *x2, void *x2norm, const void *x,
                                   const void *f, const float *w, float alpha, float eps) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(x2 && x2norm && x && f && w, "%s: null pointer", __func__);
    TRY(check_host_shape(__func__, dtype, B, C, S));
    const size_t item = (size_t)C * S * dtype_size(dtype);
    HostTensors ht;
    ht.n_in = 2; ht.in[0] = x; ht.in[1] = f; ht.in_item[0] = ht.in_item[1] = item;
    ht.n_out = 2; ht.out[0] = x2; ht.out[1] = x2norm; ht.out_item[0] = ht.out_item[1] = item;
    char *ex = nullptr;
    bool first = true;
    return run_pipelined((size_t)B, ht, (size_t)C * 4, &ex, [&](cudaStream_t st, size_t n, void **di, void **dout_) -> int {
        if (first) { ANE_CUDA_TRY(cudaMemcpyAsync(ex, w, (size_t)C * 4, cudaMemcpyHostToDevice, st)); first = false; }
        return ane_cuda_residual_rmsnorm_dev(st, dtype, (int)n, C, S, dout_[0], dout_[1], di[0], di[1], reinterpret_cast<float *>(ex), alpha, eps);
    });
}

// Flat operators: an item is a block of 64 Ki elements (the last block may be short).
static int flat_host(ane_dtype dtype, size_t n, int n_in, const void *const *in, int n_out, void *const *out, int op, float alpha) {
    const size_t esz = dtype_size(dtype);
    const size_t blk = (size_t)64 << 10;
    const size_t full = n / blk, tail = n % blk;
    for (int pass = 0; pass < 2; pass++) {
        const size_t items = pass == 0 ? full : (tail ? 1 : 0);
        if (!items) continue;
        const size_t item_elems = pass == 0 ? blk : tail;
        const size_t off = pass == 0 ? 0 : full * blk * esz;
        HostTensors ht;
        ht.n_in = n_in; ht.n_out = n_out;
        for (int i = 0; i < n_in; i++) { ht.in[i] = static_cast<const char *>(in[i]) + off; ht.in_item[i] = item_elems * esz; }
        for (int i = 0; i < n_out; i++) { ht.out[i] = static_cast<char *>(out[i]) + off; ht.out_item[i] = item_elems * esz; }
        TRY(run_pipelined(items, ht, 0, nullptr, [&](cudaStream_t st, size_t k, void **di, void **dout_) -> int {
            const size_t ne = k * item_elems;
            switch (op) {
                case 0: return ane_cuda_residual_dev(st, dtype, ne, dout_[0], di[0], di[1], alpha);
                case 1: return ane_cuda_swiglu_dev(st, dtype, ne, dout_[0], di[0], di[1]);
                default: return ane_cuda_swiglu_bwd_dev(st, dtype, ne, dout_[0], dout_[1], di[0], di[1], di[2]);
            }
        }));
    }
    return ANE_CUDA_OK;
}

int ane_cuda_residual_host(ane_dtype dtype, size_t n, void *out, const void *x, const void *f, float alpha) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && x && f && dtype_ok(dtype), "%s: bad argument", __func__);
    if (n == 0) return ANE_CUDA_OK;
    const void *in[2] = {x, f};
    void *o[1] = {out};
    return flat_host(dtype, n, 2, in, 1, o, 0, alpha);
}

int ane_cuda_swiglu_host(ane_dtype dtype, size_t n, void *out, const void *h1, const void *h3) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && h1 && h3 && dtype_ok(dtype), "%s: bad argument", __func__);
    if (n == 0) return ANE_CUDA_OK;
    const void *in[2] = {h1, h3};
    void *o[1] = {out};
    return flat_host(dtype, n, 2, in, 1, o, 1, 0.0f);
}

int ane_cuda_swiglu_bwd_host(ane_dtype dtype, size_t n, void *dh1, void *dh3, const void *h1, const void *h3, const void *dsilu) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dh1 && dh3 && h1 && h3 && dsilu && dtype_ok(dtype), "%s: bad argument", __func__);
    if (n == 0) return ANE_CUDA_OK;
    const void *in[3] = {h1, h3, dsilu};
    void *o[2] = {dh1, dh3};
    return flat_host(dtype, n, 3, in, 2, o, 2, 0.0f);
}

int ane_cuda_rope_host(ane_dtype dtype, int B, int C, int S, int hd, void *out, const void *x, float base, int pos0, unsigned flags) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && x, "%s: null pointer", __func__);
    TRY(check_host_shape(__func__, dtype, B, C, S));
    const size_t item = (size_t)C * S * dtype_size(dtype);
    HostTensors ht;
    ht.n_in = 1; ht.in[0] = x; ht.in_item[0] = item;
    ht.n_out = 1; ht.out[0] = out; ht.out_item[0] = item;
    return run_pipelined((size_t)B, ht, 0, nullptr, [&](cudaStream_t st, size_t n, void **di, void **dout_) -> int {
        return ane_cuda_rope_dev(st, dtype, (int)n, C, S, hd, dout_[0], di[0], base, pos0, flags);
    });
}

int ane_cuda_qknorm_rope_host(ane_dtype dtype, int B, int heads, int hd, int S, void *out, const void *x, const float *w,
                              float eps, float base, int pos0) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && x && w, "%s: null pointer", __func__);
    TRY(check_host_shape(__func__, dtype, B, (long long)heads * hd, S));
    const size_t item = (size_t)heads * hd * S * dtype_size(dtype);
    HostTensors ht;
    ht.n_in = 1; ht.in[0] = x; ht.in_item[0] = item;
    ht.n_out = 1; ht.out[0] = out; ht.out_item[0] = item;
    char *ex = nullptr;
    bool first = true;
    return run_pipelined((size_t)B, ht, (size_t)hd * 4, &ex, [&](cudaStream_t st, size_t n, void **di, void **dout_) -> int {
        if (first) { ANE_CUDA_TRY(cudaMemcpyAsync(ex, w, (size_t)hd * 4, cudaMemcpyHostToDevice, st)); first = false; }
        return ane_cuda_qknorm_rope_dev(st, dtype, (int)n, heads, hd, S, dout_[0], di[0], reinterpret_cast<float *>(ex), eps, base, pos0);
    });
}

int ane_cuda_rope_qknorm_bwd_host(ane_dtype dtype, int B, int heads, int hd, int S, void *dx, float *dw, const void *dy,
                                  const void *x, const float *w, float eps, float base, int pos0, unsigned flags) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dx && dw && dy && x && w, "%s: null pointer", __func__);
    TRY(check_host_shape(__func__, dtype, B, (long long)heads * hd, S));
    const size_t item = (size_t)heads * hd * S * dtype_size(dtype);
    HostTensors ht;
    ht.n_in = 2; ht.in[0] = dy; ht.in[1] = x; ht.in_item[0] = ht.in_item[1] = item;
    ht.n_out = 1; ht.out[0] = dx; ht.out_item[0] = item;
    char *ex = nullptr;
    bool first = true;
    const size_t wb = pad((size_t)hd * 4);
    cudaStream_t kst = nullptr;
    int rc = run_pipelined((size_t)B, ht, 2 * wb, &ex, [&](cudaStream_t st, size_t n, void **di, void **dout_) -> int {
        float *dw_w = reinterpret_cast<float *>(ex), *dw_dw = reinterpret_cast<float *>(ex + wb);
        if (first) {
            ANE_CUDA_TRY(cudaMemcpyAsync(dw_w, w, (size_t)hd * 4, cudaMemcpyHostToDevice, st));
            ANE_CUDA_TRY(cudaMemcpyAsync(dw_dw, dw, (size_t)hd * 4, cudaMemcpyHostToDevice, st));
            first = false;
            kst = st;
        }
        return ane_cuda_rope_qknorm_bwd_dev(st, dtype, (int)n, heads, hd, S, dout_[0], dw_dw, di[0], di[1], dw_w, eps, base, pos0, flags);
    });
    if (rc != ANE_CUDA_OK) return rc;
    ANE_CUDA_TRY(cudaMemcpyAsync(dw, ex + wb, (size_t)hd * 4, cudaMemcpyDeviceToHost, kst));
    ANE_CUDA_TRY(cudaStreamSynchronize(kst));
    return ANE_CUDA_OK;
}

// ===================================================================== reference-signature drop-ins
// fp32, one sequence, the literals of the reference (eps 1e-5, base 10000).
int ane_cuda_rmsnorm(float *out, const float *x, const float *w, int d, int S) {
    return ane_cuda_rmsnorm_host(ANE_F32, 1, d, S, out, x, w, 1e-5f);                 // eps literal of stories_cpu_ops.h:13
}

int ane_cuda_rmsnorm_bwd(float *dx, float *dw, const float *dy, const float *x, const float *w, int d, int S) {
    return ane_cuda_rmsnorm_bwd_host(ANE_F32, 1, d, S, dx, dw, dy, x, w, nullptr, 1e-5f, ANE_NORM_BWD_REFERENCE);
}

int ane_cuda_rope_backward_inplace(float *dx, int seq, int dim, int hd) {
    return ane_cuda_rope_host(ANE_F32, 1, dim, seq, hd, dx, dx, 10000.0f, 0, ANE_ROPE_INVERSE);   // base literal of cpu_ops.h:172
}

int ane_cuda_residual(float *out, const float *x, const float *f, float alpha, size_t n) {
    return ane_cuda_residual_host(ANE_F32, n, out, x, f, alpha);
}

int ane_cuda_swiglu(float *out, const float *h1, const float *h3, size_t n) {
    return ane_cuda_swiglu_host(ANE_F32, n, out, h1, h3);
}

int ane_cuda_swiglu_bwd(float *dh1, float *dh3, const float *h1, const float *h3, const float *dsilu, size_t n) {
    return ane_cuda_swiglu_bwd_host(ANE_F32, n, dh1, dh3, h1, h3, dsilu);
}

static int adam_host(float *w, const float *g, AdamState *st, int t, float lr, float b1, float b2, float eps, float wd, unsigned variant) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(w && g && st && st->m && st->v, "adam_update: null pointer");
    const size_t n = st->n;
    if (n == 0) return ANE_CUDA_OK;
    const size_t blk = (size_t)64 << 10;
    const size_t full = n / blk, tail = n % blk;
    for (int pass = 0; pass < 2; pass++) {
        const size_t items = pass == 0 ? full : (tail ? 1 : 0);
        if (!items) continue;
        const size_t ie = pass == 0 ? blk : tail;
        const size_t off = pass == 0 ? 0 : full * blk;
        HostTensors ht;
        ht.n_in = 4; ht.n_out = 3;
        ht.in[0] = w + off; ht.in[1] = g + off; ht.in[2] = st->m + off; ht.in[3] = st->v + off;
        ht.out[0] = w + off; ht.out[1] = st->m + off; ht.out[2] = st->v + off;
        for (int i = 0; i < 4; i++) ht.in_item[i] = ie * 4;
        for (int i = 0; i < 3; i++) ht.out_item[i] = ie * 4;
        TRY(run_pipelined(items, ht, 0, nullptr, [&](cudaStream_t s, size_t k, void **di, void **dout_) -> int {
            const size_t ne = k * ie;
            // update in place in the input slot, then copy the three results to the output slot
            TRY(ane_cuda_adam_dev(s, ne, (float *)di[0], (const float *)di[1], (float *)di[2], (float *)di[3], t, lr, b1, b2, eps, wd, 1.0f, nullptr, variant));
            ANE_CUDA_TRY(cudaMemcpyAsync(dout_[0], di[0], ne * 4, cudaMemcpyDeviceToDevice, s));
            ANE_CUDA_TRY(cudaMemcpyAsync(dout_[1], di[2], ne * 4, cudaMemcpyDeviceToDevice, s));
            ANE_CUDA_TRY(cudaMemcpyAsync(dout_[2], di[3], ne * 4, cudaMemcpyDeviceToDevice, s));
            return ANE_CUDA_OK;
        }));
    }
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

}  // extern "C"
