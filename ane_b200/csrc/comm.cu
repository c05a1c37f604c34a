// comm.cu -- the multi-GPU group of the C ABI: one process per GPU, NCCL as the transport.
//
// The operator chain itself needs no exchange (sequences are sharded, every operator is per token).  What a
// data-parallel step exchanges is: the scalar loss (ane_cuda_allreduce_f32), and the optimizer step over the flat
// parameter space (ane_cuda_sharded_adam_step; the reference's single-process form is the Adam loop of
// training_dynamic/train.m:837-869 after the scale / norm / clip of :750-825):
//     reduce-scatter of the gradients -> squared norm of the slice -> all-reduce of the scalar -> clip factor ->
//     Adam on the rank's slice (weight decay on [0, n_decay) only) -> all-gather of the parameters.
// Two transports compute the same step: NCCL collectives, or -- after ane_cuda_comm_map_peers -- this library's own
// kernels on peer-mapped buffers (p2p.cu): the reduce kernel reads every rank's gradients over NVLink with plain
// loads, the Adam kernel stores the new weights to every rank, and one-element all-reduces order the phases, so no
// kernel ever waits for another rank.
//
// NCCL is loaded at run time (dlopen of libnccl.so.2) so that the library loads on machines without it.
// Every host-side wait polls the stream and the communicator against a deadline and returns ANE_CUDA_ERR_TIMEOUT
// after aborting the communicator; nothing here spins on the device.
#include "common.cuh"

#include <cuda.h>
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <thread>
#include <vector>

namespace ane {

struct NcclApi {
    void *so = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};
static NcclApi g_nccl;

static int nccl_load() {
    if (g_nccl.so) return ANE_CUDA_OK;
    void *so = nullptr;
    for (const char *name : {"libnccl.so.2", "libnccl.so"}) {
        so = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
        if (so) break;
    }
    if (!so) return fail(ANE_CUDA_ERR_UNSUPPORTED, "multi-GPU group: cannot load libnccl.so.2 (%s)", dlerror());
    NcclApi a;
    a.so = so;
#define ANE_SYM(field, sym)                                                                                              \
    a.field = reinterpret_cast<decltype(a.field)>(dlsym(so, sym));                                                      \
    if (!a.field) { dlclose(so); return fail(ANE_CUDA_ERR_UNSUPPORTED, "multi-GPU group: libnccl lacks %s", sym); }
    ANE_SYM(GetUniqueId, "ncclGetUniqueId")
    ANE_SYM(CommInitRankConfig, "ncclCommInitRankConfig")
    ANE_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
    ANE_SYM(CommAbort, "ncclCommAbort")
    ANE_SYM(CommDestroy, "ncclCommDestroy")
    ANE_SYM(AllReduce, "ncclAllReduce")
    ANE_SYM(ReduceScatter, "ncclReduceScatter")
    ANE_SYM(AllGather, "ncclAllGather")
    ANE_SYM(GetErrorString, "ncclGetErrorString")
#undef ANE_SYM
    g_nccl = a;
    return ANE_CUDA_OK;
}

struct PeerMap { float *w[ANE_CUDA_MAX_RANKS]; float *g[ANE_CUDA_MAX_RANKS]; void *opened[2 * ANE_CUDA_MAX_RANKS]; int nopened; bool on; const float *w_self, *g_self; };

struct Comm {
    ncclComm_t comm = nullptr;
    int nranks = 0, rank = -1;
    double timeout_s = 30.0;
    float *g_slice = nullptr;      // the rank's reduced gradient slice
    size_t g_slice_floats = 0;
    float *scalars = nullptr;      // [0..1] squared-norm partials, [2] clip factor, [3] rank-sync token, [4..] reduce block partials
    PeerMap peers = {};
};
static Comm g_comm;
constexpr size_t COMM_SCALARS = 8 + 1184;

using Clock = std::chrono::steady_clock;

__global__ void comm_sum2_kernel(float *out, const float *a) { out[0] = a[0] + a[1]; }

static int nccl_fail(const char *what, ncclResult_t r) {
    return fail(ANE_CUDA_ERR_CUDA, "%s: NCCL error %d (%s)", what, (int)r, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?");
}

static void comm_abort() {
    if (g_comm.comm) { g_nccl.CommAbort(g_comm.comm); g_comm.comm = nullptr; }
}

// Polls until the communicator's pending operation has finished (ncclSuccess), failed, or the deadline passes.
static int wait_comm_ready(const char *what, double timeout_s) {
    const auto deadline = Clock::now() + std::chrono::duration<double>(timeout_s);
    for (;;) {
        ncclResult_t st = ncclSuccess;
        const ncclResult_t r = g_nccl.CommGetAsyncError(g_comm.comm, &st);
        if (r != ncclSuccess) { comm_abort(); return nccl_fail(what, r); }
        if (st == ncclSuccess) return ANE_CUDA_OK;
        if (st != ncclInProgress) { comm_abort(); return nccl_fail(what, st); }
        if (Clock::now() >= deadline) {
            comm_abort();
            return fail(ANE_CUDA_ERR_TIMEOUT, "%s: not complete after %.3f s (a rank that never joined?); the communicator was aborted", what, timeout_s);
        }
        std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
}

#define ANE_NCCL_TRY(what, expr)                                                                                         \
    do {                                                                                                                 \
        ncclResult_t r__ = (expr);                                                                                       \
        if (r__ == ncclInProgress) { if (int rc__ = wait_comm_ready(what, g_comm.timeout_s)) return rc__; }               \
        else if (r__ != ncclSuccess) return nccl_fail(what, r__);                                                         \
    } while (0)

static int require_comm(const char *fn) {
    if (!ctx().inited) return fail(ANE_CUDA_ERR_NOT_INIT, "%s: call ane_cuda_init first", fn);
    if (!g_comm.comm) return fail(ANE_CUDA_ERR_NOT_INIT, "%s: call ane_cuda_comm_init first", fn);
    return ANE_CUDA_OK;
}

static int stream_wait(const char *fn, cudaStream_t st, double timeout_s) {
    const auto deadline = Clock::now() + std::chrono::duration<double>(timeout_s);
    for (;;) {
        const cudaError_t q = cudaStreamQuery(st);
        if (q == cudaSuccess) return ANE_CUDA_OK;
        if (q != cudaErrorNotReady) { cudaGetLastError(); return fail(ANE_CUDA_ERR_CUDA, "%s: stream failed: %s", fn, cudaGetErrorString(q)); }
        if (g_comm.comm) {
            ncclResult_t as = ncclSuccess;
            if (g_nccl.CommGetAsyncError(g_comm.comm, &as) == ncclSuccess && as != ncclSuccess && as != ncclInProgress) {
                comm_abort();
                return nccl_fail(fn, as);
            }
        }
        if (Clock::now() >= deadline) {
            comm_abort();      // unblocks a collective kernel that waits for a rank which will not come
            return fail(ANE_CUDA_ERR_TIMEOUT, "%s: work on the stream not complete after %.3f s; the communicator was aborted", fn, timeout_s);
        }
        std::this_thread::sleep_for(std::chrono::microseconds(100));
    }
}

static void peers_close() {
    for (int i = 0; i < g_comm.peers.nopened; i++) cudaIpcCloseMemHandle(g_comm.peers.opened[i]);
    g_comm.peers = PeerMap();
}

}  // namespace ane

using namespace ane;

extern "C" {

int ane_cuda_comm_unique_id(void *id_out) {
    ANE_REQUIRE(id_out, "%s: null pointer", __func__);
    if (int rc = nccl_load()) return rc;
    static_assert(sizeof(ncclUniqueId) == ANE_CUDA_COMM_ID_BYTES, "ncclUniqueId is 128 bytes");
    ncclUniqueId id;
    const ncclResult_t r = g_nccl.GetUniqueId(&id);
    if (r != ncclSuccess) return nccl_fail(__func__, r);
    memcpy(id_out, &id, sizeof(id));
    return ANE_CUDA_OK;
}

int ane_cuda_comm_init(int nranks, int rank, const void *id, double timeout_s) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(id, "%s: null pointer", __func__);
    ANE_REQUIRE(nranks >= 1 && nranks <= ANE_CUDA_MAX_RANKS && rank >= 0 && rank < nranks, "%s: bad rank %d of %d (at most %d ranks)", __func__, rank,
                nranks, ANE_CUDA_MAX_RANKS);
    ANE_REQUIRE(timeout_s >= 0.0, "%s: negative timeout", __func__);
    if (g_comm.comm) return fail(ANE_CUDA_ERR_INVALID, "%s: a communicator already exists (ane_cuda_comm_destroy first)", __func__);
    if (int rc = nccl_load()) return rc;
    ncclUniqueId uid;
    memcpy(&uid, id, sizeof(uid));
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    cfg.blocking = 0;                                  // every call returns at once; completion is polled against a deadline
    g_comm.timeout_s = timeout_s;
    g_comm.nranks = nranks;
    g_comm.rank = rank;
    const ncclResult_t r = g_nccl.CommInitRankConfig(&g_comm.comm, nranks, uid, rank, &cfg);
    if (r != ncclSuccess && r != ncclInProgress) { g_comm.comm = nullptr; return nccl_fail(__func__, r); }
    if (int rc = wait_comm_ready(__func__, timeout_s)) return rc;
    if (!g_comm.scalars) {
        if (dev_malloc(reinterpret_cast<void **>(&g_comm.scalars), COMM_SCALARS * sizeof(float)) != cudaSuccess) {
            comm_abort();
            return fail(ANE_CUDA_ERR_NOMEM, "%s: no device memory for the scalars", __func__);
        }
        cudaMemset(g_comm.scalars, 0, COMM_SCALARS * sizeof(float));
    }
    return ANE_CUDA_OK;
}

int ane_cuda_comm_size(void) { return g_comm.comm ? g_comm.nranks : 0; }
int ane_cuda_comm_rank(void) { return g_comm.comm ? g_comm.rank : -1; }

int ane_cuda_comm_destroy(void) {
    peers_close();
    if (g_comm.comm) {
        cudaDeviceSynchronize();
        g_nccl.CommDestroy(g_comm.comm);
        g_comm.comm = nullptr;
    }
    if (g_comm.g_slice) cudaFree(g_comm.g_slice);
    if (g_comm.scalars) cudaFree(g_comm.scalars);
    g_comm = Comm();
    return ANE_CUDA_OK;
}

int ane_cuda_comm_wait(void *stream, double timeout_s) {
    ANE_REQUIRE_INIT();
    return stream_wait(__func__, (cudaStream_t)stream, timeout_s < 0 ? g_comm.timeout_s : timeout_s);
}

int ane_cuda_allreduce_f32(void *stream, float *buf, size_t n) {
    if (int rc = require_comm(__func__)) return rc;
    ANE_REQUIRE(buf || n == 0, "%s: null pointer", __func__);
    if (n == 0) return ANE_CUDA_OK;
    ANE_NCCL_TRY(__func__, g_nccl.AllReduce(buf, buf, n, ncclFloat, ncclSum, g_comm.comm, (cudaStream_t)stream));
    return ANE_CUDA_OK;
}

// Exchanges CUDA IPC handles of the flat parameter and gradient buffers so that every rank can address every other
// rank's copy; collective and blocking (it ends with a deadline-bounded wait).
int ane_cuda_comm_map_peers(float *w, float *g, size_t n_floats) {
    if (int rc = require_comm(__func__)) return rc;
    ANE_REQUIRE(w && g && n_floats > 0, "%s: null pointer", __func__);
    peers_close();
    struct Rec { cudaIpcMemHandle_t hw, hg; unsigned long long off_w, off_g, bytes; unsigned long long pad; };
    static_assert(sizeof(Rec) % 16 == 0, "records are gathered as bytes");
    Rec mine;
    memset(&mine, 0, sizeof(mine));
    void *base_w = nullptr, *base_g = nullptr;
    {   // a handle names a whole allocation: find its base
        typedef CUresult (*RangeFn)(CUdeviceptr *, size_t *, CUdeviceptr);
        static RangeFn range = nullptr;
        if (!range) {
            cudaDriverEntryPointQueryResult qr;
            void *fn = nullptr;
            if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qr) != cudaSuccess || !fn) {
                cudaGetLastError();
                return fail(ANE_CUDA_ERR_UNSUPPORTED, "%s: cuMemGetAddressRange unavailable", __func__);
            }
            range = reinterpret_cast<RangeFn>(fn);
        }
        CUdeviceptr b = 0;
        size_t sz = 0;
        if (range(&b, &sz, (CUdeviceptr)w) != CUDA_SUCCESS) return fail(ANE_CUDA_ERR_INVALID, "%s: w is not device memory", __func__);
        base_w = (void *)b;
        if (range(&b, &sz, (CUdeviceptr)g) != CUDA_SUCCESS) return fail(ANE_CUDA_ERR_INVALID, "%s: g is not device memory", __func__);
        base_g = (void *)b;
    }
    cudaError_t e = cudaIpcGetMemHandle(&mine.hw, base_w);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&mine.hg, base_g);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(ANE_CUDA_ERR_UNSUPPORTED, "%s: cudaIpcGetMemHandle failed: %s", __func__, cudaGetErrorString(e)); }
    mine.off_w = (unsigned long long)((char *)w - (char *)base_w);
    mine.off_g = (unsigned long long)((char *)g - (char *)base_g);
    mine.bytes = n_floats * sizeof(float);
    const int N = g_comm.nranks;
    Rec *dev = nullptr;
    if (dev_malloc(reinterpret_cast<void **>(&dev), sizeof(Rec) * N) != cudaSuccess) return fail(ANE_CUDA_ERR_NOMEM, "%s: no device memory", __func__);
    std::vector<Rec> all(N);
    int rc = ANE_CUDA_OK;
    do {
        if (cudaMemcpy(dev + g_comm.rank, &mine, sizeof(Rec), cudaMemcpyHostToDevice) != cudaSuccess) { rc = fail(ANE_CUDA_ERR_CUDA, "%s: copy failed", __func__); break; }
        ncclResult_t r = g_nccl.AllGather(dev + g_comm.rank, dev, sizeof(Rec), ncclChar, g_comm.comm, nullptr);
        if (r == ncclInProgress) rc = wait_comm_ready(__func__, g_comm.timeout_s);
        else if (r != ncclSuccess) rc = nccl_fail(__func__, r);
        if (rc) break;
        rc = stream_wait(__func__, nullptr, g_comm.timeout_s);
        if (rc) break;
        if (cudaMemcpy(all.data(), dev, sizeof(Rec) * N, cudaMemcpyDeviceToHost) != cudaSuccess) { rc = fail(ANE_CUDA_ERR_CUDA, "%s: copy failed", __func__); break; }
    } while (0);
    cudaFree(dev);
    if (rc) return rc;
    PeerMap &pm = g_comm.peers;
    for (int r = 0; r < N; r++) {
        if (all[r].bytes != mine.bytes) { peers_close(); return fail(ANE_CUDA_ERR_INVALID, "%s: rank %d registered %llu bytes, this rank %llu", __func__, r, all[r].bytes, mine.bytes); }
        if (r == g_comm.rank) { pm.w[r] = w; pm.g[r] = g; continue; }
        void *pw = nullptr, *pg = nullptr;
        e = cudaIpcOpenMemHandle(&pw, all[r].hw, cudaIpcMemLazyEnablePeerAccess);
        if (e == cudaSuccess) { pm.opened[pm.nopened++] = pw; e = cudaIpcOpenMemHandle(&pg, all[r].hg, cudaIpcMemLazyEnablePeerAccess); }
        if (e == cudaSuccess) pm.opened[pm.nopened++] = pg;
        if (e != cudaSuccess) {
            cudaGetLastError();
            peers_close();
            return fail(ANE_CUDA_ERR_UNSUPPORTED, "%s: cannot map rank %d's buffers: %s", __func__, r, cudaGetErrorString(e));
        }
        pm.w[r] = reinterpret_cast<float *>((char *)pw + all[r].off_w);
        pm.g[r] = reinterpret_cast<float *>((char *)pg + all[r].off_g);
    }
    pm.on = true;
    pm.w_self = w;
    pm.g_self = g;
    return ANE_CUDA_OK;
}

int ane_cuda_comm_unmap_peers(void) {
    if (g_comm.peers.on || g_comm.peers.nopened) { cudaDeviceSynchronize(); peers_close(); }
    return ANE_CUDA_OK;
}

int ane_cuda_sharded_adam_step(void *stream, float *w, float *g, float *m, float *v, size_t n_padded, size_t n_decay, size_t n_params,
                               int t, float lr, float b1, float b2, float eps, float wd, float gscale, float clip, unsigned flags,
                               float *normsq_out) {
    if (int rc = require_comm(__func__)) return rc;
    ANE_REQUIRE(w && g && m && v, "%s: null pointer", __func__);
    const int N = g_comm.nranks, rank = g_comm.rank;
    ANE_REQUIRE(n_padded > 0 && n_padded % (size_t)N == 0, "%s: the flat buffers must hold a multiple of %d floats (got %zu)", __func__, N, n_padded);
    ANE_REQUIRE(n_decay <= n_params && n_params <= n_padded, "%s: need n_decay <= n_params <= n_padded", __func__);
    ANE_REQUIRE(t >= 1, "%s: step t must be >= 1 (got %d)", __func__, t);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t slice = n_padded / N, lo = (size_t)rank * slice, hi = lo + slice;
    float *sc = g_comm.scalars;
    const bool peer = g_comm.peers.on && g_comm.peers.w_self == w && g_comm.peers.g_self == g && N > 1;
    float *gs = nullptr;
    if (N > 1) {
        if (g_comm.g_slice_floats < slice) {
            if (frozen()) return fail(ANE_CUDA_ERR_NOMEM, "%s: the gradient slice buffer would have to grow and the library is frozen", __func__);
            retire_device_range(g_comm.g_slice);
            g_comm.g_slice = nullptr;
            g_comm.g_slice_floats = 0;
            if (dev_malloc(reinterpret_cast<void **>(&g_comm.g_slice), slice * sizeof(float)) != cudaSuccess)
                return fail(ANE_CUDA_ERR_NOMEM, "%s: no device memory for the gradient slice (%zu floats)", __func__, slice);
            g_comm.g_slice_floats = slice;
        }
        gs = g_comm.g_slice;
    } else {
        gs = g;
    }
    if (peer) {
        ANE_CUDA_TRY(cudaMemsetAsync(sc, 0, 2 * sizeof(float), st));
        ANE_NCCL_TRY(__func__, g_nccl.AllReduce(sc + 3, sc + 3, 1, ncclFloat, ncclSum, g_comm.comm, st));      // every rank's gradients are complete
        if (int rc = ane_cuda_p2p_reduce_dev(st, N, g_comm.peers.g, lo, slice, gs, gscale, sc + 1, sc + 8)) return rc;
        ANE_NCCL_TRY(__func__, g_nccl.AllReduce(sc, sc, 2, ncclFloat, ncclSum, g_comm.comm, st));              // the norm; all reads of gradients done
        if (int rc = ane_cuda_clip_factor_dev(st, sc, 2, clip, sc + 2)) return rc;
    } else {
        if (N > 1) ANE_NCCL_TRY(__func__, g_nccl.ReduceScatter(g, gs, slice, ncclFloat, ncclSum, g_comm.comm, st));
        if (int rc = ane_cuda_grad_norm_sq_dev(st, slice, N > 1 ? gs : g + lo, gscale, sc)) return rc;
        if (N > 1) ANE_NCCL_TRY(__func__, g_nccl.AllReduce(sc, sc, 1, ncclFloat, ncclSum, g_comm.comm, st));
        if (int rc = ane_cuda_clip_factor_dev(st, sc, 1, clip, sc + 2)) return rc;
    }
    const size_t ranges[2][2] = {{0, n_decay}, {n_decay, n_params}};
    for (int k = 0; k < 2; k++) {
        const size_t a = ranges[k][0] > lo ? ranges[k][0] : lo, b = ranges[k][1] < hi ? ranges[k][1] : hi;
        if (a >= b) continue;
        const float wdk = k == 0 ? wd : 0.0f;            // norm weights take no decay (train.m:852-869)
        const float *gk = (N > 1 ? gs : g + lo) + (a - lo);
        int rc;
        if (peer) rc = ane_cuda_p2p_adam_dev(st, N, rank, g_comm.peers.w, a, b - a, gk, m + a, v + a, t, lr, b1, b2, eps, wdk, gscale, sc + 2, flags);
        else rc = ane_cuda_adam_dev(st, b - a, w + a, gk, m + a, v + a, t, lr, b1, b2, eps, wdk, gscale, sc + 2, flags);
        if (rc) return rc;
    }
    if (peer) {
        ANE_NCCL_TRY(__func__, g_nccl.AllReduce(sc + 3, sc + 3, 1, ncclFloat, ncclSum, g_comm.comm, st));      // every rank's parameter stores have landed
    } else if (N > 1) {
        ANE_NCCL_TRY(__func__, g_nccl.AllGather(w + lo, w, slice, ncclFloat, g_comm.comm, st));
    }
    if (normsq_out) {
        // one float: the global squared gradient norm of this step (sum of the partials in peer mode)
        if (peer) { comm_sum2_kernel<<<1, 1, 0, st>>>(normsq_out, sc); ANE_LAUNCH_OK(1); }
        else ANE_CUDA_TRY(cudaMemcpyAsync(normsq_out, sc, sizeof(float), cudaMemcpyDeviceToDevice, st));
    }
    return ANE_CUDA_OK;
}

}  // extern "C"
