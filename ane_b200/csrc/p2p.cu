// p2p.cu -- the sharded optimizer step with its two collectives folded into the kernels, over peer memory.
//
// Data-parallel ranks each hold a full flat gradient buffer g_r and a full flat parameter buffer w_r; rank k
// owns the slice [lo, lo + n) of the optimizer state (ZeRO-1).  With every rank's buffers mapped into every
// other rank's address space (CUDA IPC / symmetric memory over NVLink) the step is two kernels per rank:
//
//   reduce     gs[i] = g_0[lo+i] + g_1[lo+i] + ... (fixed rank order: the same bits on every run and for any
//              assignment of slices), read straight from the peers' memory -- the reduce-scatter -- and the
//              block partials of sum((gs*gscale)^2) for the clipping norm in the same pass;
//   update     Adam on the slice (same arithmetic and association order as ane_cuda_adam_dev), the new
//              weights stored to the slice position of EVERY rank's parameter buffer -- the all-gather.
//
// No kernel here waits for another rank: the caller orders the phases across ranks on the stream (any
// collective all ranks take part in -- in practice the scalar all-reduce of the clipping norm and a
// one-element all-reduce -- is such an ordering point), so nothing can spin.  Loads and stores to peers are
// plain 16-byte accesses; no TMA, no multicast.
#include "common.cuh"

#include <math.h>

namespace ane {

constexpr int P2P_MAX_RANKS = 8;
constexpr int P2P_THREADS = 256;
constexpr int P2P_MAX_BLOCKS = 1184;      // 148 SMs x 8

struct PeerConst { const float *p[P2P_MAX_RANKS]; };
struct PeerMut { float *p[P2P_MAX_RANKS]; };

// Block b owns the contiguous chunk [b*chunk, (b+1)*chunk) of the slice: its partial sum of squares depends on
// (n, gridDim) only, not on scheduling.
__global__ void __launch_bounds__(P2P_THREADS)
p2p_reduce_kernel(float *__restrict__ gs, float *__restrict__ partial, PeerConst g, int nranks, size_t lo, size_t n, float gscale) {
    const size_t chunk = ((n + gridDim.x - 1) / gridDim.x + 3) & ~(size_t)3;
    const size_t b0 = (size_t)blockIdx.x * chunk;
    const size_t b1 = b0 + chunk < n ? b0 + chunk : n;
    float acc = 0.0f;
    if (b0 < b1) {
        bool al = (reinterpret_cast<uintptr_t>(gs) & 15u) == 0 && (lo & 3) == 0;
        for (int r = 0; r < nranks; r++) al = al && (reinterpret_cast<uintptr_t>(g.p[r]) & 15u) == 0;
        size_t done = b0;
        if (al) {
            const size_t nv = (b1 - b0) / 4;
            for (size_t i = threadIdx.x; i < nv; i += P2P_THREADS) {
                const size_t e = b0 + i * 4;
                float4 s = __ldcs(reinterpret_cast<const float4 *>(g.p[0] + lo + e));
                for (int r = 1; r < nranks; r++) {
                    const float4 q = __ldcs(reinterpret_cast<const float4 *>(g.p[r] + lo + e));
                    s.x = __fadd_rn(s.x, q.x); s.y = __fadd_rn(s.y, q.y); s.z = __fadd_rn(s.z, q.z); s.w = __fadd_rn(s.w, q.w);
                }
                *reinterpret_cast<float4 *>(gs + e) = s;
                const float a = s.x * gscale, b = s.y * gscale, c = s.z * gscale, d = s.w * gscale;
                acc += a * a; acc += b * b; acc += c * c; acc += d * d;
            }
            done = b0 + nv * 4;
        }
        for (size_t e = done + threadIdx.x; e < b1; e += P2P_THREADS) {
            float s = g.p[0][lo + e];
            for (int r = 1; r < nranks; r++) s = __fadd_rn(s, g.p[r][lo + e]);
            gs[e] = s;
            const float a = s * gscale;
            acc += a * a;
        }
    }
    __shared__ float sh[P2P_THREADS / 32];
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int i = 0; i < P2P_THREADS / 32; i++) s += sh[i];
        partial[blockIdx.x] = s;
    }
}

__global__ void p2p_sum_partials_kernel(const float *__restrict__ partial, int nblocks, float *__restrict__ out) {
    float acc = 0.0f;        // one warp, fixed order
    for (int i = threadIdx.x; i < nblocks; i += 32) acc += partial[i];
    acc = warp_sum(acc);
    if (threadIdx.x == 0) *out = acc;
}

struct AdamConsts {
    float b1, b2, omb1, omb2, bc1, bc2, lr, eps, wd, gscale;
    const float *clip;
    unsigned variant;
    bool use_gscale;
};

// stories_cpu_ops.h:55-63 / training_dynamic/cpu_ops.h:56-64, the association order of AdamOp (elementwise.cu)
__device__ __forceinline__ float adam_one(float w, float g, float &m, float &v, const AdamConsts &c, float clipf) {
    if (c.use_gscale) g = __fmul_rn(g, c.gscale);
    if (c.clip) g = __fmul_rn(g, clipf);
    m = __fadd_rn(__fmul_rn(c.b1, m), __fmul_rn(c.omb1, g));
    v = __fadd_rn(__fmul_rn(c.b2, v), __fmul_rn(__fmul_rn(c.omb2, g), g));
    const float mh = __fdiv_rn(m, c.bc1), vh = __fdiv_rn(v, c.bc2);
    const float den = __fadd_rn(__fsqrt_rn(vh), c.eps);
    if (c.variant == ANE_ADAM_STORIES) return __fsub_rn(w, __fdiv_rn(__fmul_rn(c.lr, mh), den));
    return __fsub_rn(w, __fmul_rn(c.lr, __fadd_rn(__fdiv_rn(mh, den), __fmul_rn(c.wd, w))));
}

// w_all.p[r] = rank r's FULL parameter buffer; w_all.p[self] is read.  m, v, gs are the owner's slice-sized arrays.
__global__ void __launch_bounds__(P2P_THREADS)
p2p_adam_kernel(PeerMut w_all, int nranks, int self, size_t lo, size_t n, const float *__restrict__ gs, float *__restrict__ m,
                float *__restrict__ v, AdamConsts c) {
    const float clipf = c.clip ? __ldg(c.clip) : 1.0f;
    bool al = (lo & 3) == 0 && ((reinterpret_cast<uintptr_t>(gs) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15u) == 0;
    for (int r = 0; r < nranks; r++) al = al && (reinterpret_cast<uintptr_t>(w_all.p[r]) & 15u) == 0;
    const size_t gsz = (size_t)gridDim.x * P2P_THREADS, tid = (size_t)blockIdx.x * P2P_THREADS + threadIdx.x;
    size_t done = 0;
    if (al) {
        const size_t nv = n / 4;
        for (size_t i = tid; i < nv; i += gsz) {
            const size_t e = i * 4;
            const float4 w4 = *reinterpret_cast<const float4 *>(w_all.p[self] + lo + e);
            const float4 g4 = __ldcs(reinterpret_cast<const float4 *>(gs + e));
            float4 m4 = *reinterpret_cast<const float4 *>(m + e), v4 = *reinterpret_cast<const float4 *>(v + e);
            float4 o;
            o.x = adam_one(w4.x, g4.x, m4.x, v4.x, c, clipf);
            o.y = adam_one(w4.y, g4.y, m4.y, v4.y, c, clipf);
            o.z = adam_one(w4.z, g4.z, m4.z, v4.z, c, clipf);
            o.w = adam_one(w4.w, g4.w, m4.w, v4.w, c, clipf);
            *reinterpret_cast<float4 *>(m + e) = m4;
            *reinterpret_cast<float4 *>(v + e) = v4;
            for (int r = 0; r < nranks; r++) *reinterpret_cast<float4 *>(w_all.p[r] + lo + e) = o;
        }
        done = nv * 4;
    }
    for (size_t e = done + tid; e < n; e += gsz) {
        float mm = m[e], vv = v[e];
        const float o = adam_one(w_all.p[self][lo + e], gs[e], mm, vv, c, clipf);
        m[e] = mm;
        v[e] = vv;
        for (int r = 0; r < nranks; r++) w_all.p[r][lo + e] = o;
    }
}

}  // namespace ane

using namespace ane;

extern "C" {

int ane_cuda_p2p_reduce_dev(void *stream, int nranks, const float *const *g_ranks, size_t lo, size_t n, float *g_slice, float gscale,
                            float *normsq_dev, float *scratch) {
    return ane_cuda_p2p_reduce_limited_dev(stream, nranks, g_ranks, lo, n, g_slice, gscale, normsq_dev, scratch, 0);
}

int ane_cuda_p2p_reduce_limited_dev(void *stream, int nranks, const float *const *g_ranks, size_t lo, size_t n, float *g_slice, float gscale,
                                    float *normsq_dev, float *scratch, int max_blocks) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(g_ranks && g_slice && normsq_dev, "%s: null pointer", __func__);
    ANE_REQUIRE(nranks >= 1 && nranks <= P2P_MAX_RANKS, "%s: 1..%d ranks (got %d)", __func__, P2P_MAX_RANKS, nranks);
    PeerConst g;
    for (int r = 0; r < P2P_MAX_RANKS; r++) g.p[r] = r < nranks ? g_ranks[r] : nullptr;
    for (int r = 0; r < nranks; r++) ANE_REQUIRE(g.p[r], "%s: rank %d has no buffer", __func__, r);
    size_t blocks = (n + (size_t)P2P_THREADS * 16 - 1) / ((size_t)P2P_THREADS * 16);
    if (blocks < 1) blocks = 1;
    if (blocks > P2P_MAX_BLOCKS) blocks = P2P_MAX_BLOCKS;
    if (max_blocks > 0 && blocks > (size_t)max_blocks) blocks = (size_t)max_blocks;      // a background reduce beside other kernels
    // block partials: the caller's scratch (needed when this call runs on a stream beside other operators of the
    // library, which share the library-owned range) or the library-owned range
    float *partial = scratch ? scratch : static_cast<float *>(workspace(P2P_MAX_BLOCKS * sizeof(float)));
    if (!partial) return fail(ANE_CUDA_ERR_NOMEM, "%s: no scratch", __func__);
    cudaStream_t st = (cudaStream_t)stream;
    p2p_reduce_kernel<<<(unsigned)blocks, P2P_THREADS, 0, st>>>(g_slice, partial, g, nranks, lo, n, gscale);
    p2p_sum_partials_kernel<<<1, 32, 0, st>>>(partial, (int)blocks, normsq_dev);
    ANE_LAUNCH_OK(2);
    return ANE_CUDA_OK;
}

int ane_cuda_p2p_adam_dev(void *stream, int nranks, int self, float *const *w_ranks, size_t lo, size_t n, const float *g_slice,
                          float *m_slice, float *v_slice, int t, float lr, float b1, float b2, float eps, float wd, float gscale,
                          const float *clip_dev, unsigned flags) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(w_ranks && g_slice && m_slice && v_slice, "%s: null pointer", __func__);
    ANE_REQUIRE(nranks >= 1 && nranks <= P2P_MAX_RANKS && self >= 0 && self < nranks, "%s: bad rank %d of %d", __func__, self, nranks);
    ANE_REQUIRE(t >= 1, "%s: step t must be >= 1 (got %d)", __func__, t);
    ANE_REQUIRE(flags == ANE_ADAM_STORIES || flags == ANE_ADAM_DYNAMIC, "%s: bad flags %u", __func__, flags);
    if (n == 0) return ANE_CUDA_OK;
    PeerMut w;
    for (int r = 0; r < P2P_MAX_RANKS; r++) w.p[r] = r < nranks ? w_ranks[r] : nullptr;
    for (int r = 0; r < nranks; r++) ANE_REQUIRE(w.p[r], "%s: rank %d has no buffer", __func__, r);
    AdamConsts c;
    c.b1 = b1; c.b2 = b2;
    c.omb1 = 1 - b1; c.omb2 = 1 - b2;
    c.bc1 = 1.0f - powf(b1, t);       // host libm, as the reference computes them
    c.bc2 = 1.0f - powf(b2, t);
    c.lr = lr; c.eps = eps; c.wd = wd; c.gscale = gscale;
    c.use_gscale = gscale != 1.0f;
    c.clip = clip_dev;
    c.variant = flags;
    size_t blocks = (n / 4 + P2P_THREADS - 1) / P2P_THREADS;
    if (blocks < 1) blocks = 1;
    const size_t cap = (size_t)ctx().sm_count * 8;
    if (blocks > cap) blocks = cap;
    p2p_adam_kernel<<<(unsigned)blocks, P2P_THREADS, 0, (cudaStream_t)stream>>>(w, nranks, self, lo, n, g_slice, m_slice, v_slice, c);
    ANE_LAUNCH_OK(1);
    return ANE_CUDA_OK;
}

}  // extern "C"
