// elementwise.cu -- flat streaming operators: DeepNet-alpha residual, scale, SwiGLU gate
// forward and backward, Adam, gradient norm and clip factor.
//
// Every kernel here is bound by HBM bandwidth: each element is read once and written once.
// A thread moves UNROLL 16-byte vectors per tensor; all loads of an iteration are issued
// before the first use so that each SM keeps tens of kilobytes in flight.  Streaming cache
// hints keep read-once data from displacing anything useful in L2.
#include "common.cuh"

namespace ane {

template <int NIN, int NOUT> struct EwPtrs {
    const void *in[NIN];
    void *out[NOUT];
};

constexpr int EW_THREADS = 256;
constexpr int EW_UNROLL = 4;

// Vector body: n_vec full vectors, then (block 0, thread 0) finishes the n_tail scalars.
template <typename T, int NIN, int NOUT, class Op>
__global__ void __launch_bounds__(EW_THREADS)
ew_vec_kernel(EwPtrs<NIN, NOUT> p, size_t n_vec, int n_tail, Op op) {
    constexpr int VEC = Elt<T>::VEC;
    const size_t base = (size_t)blockIdx.x * (EW_THREADS * EW_UNROLL) + threadIdx.x;
    dep_sync();
    Raw<T, VEC> r[EW_UNROLL][NIN];
#pragma unroll
    for (int u = 0; u < EW_UNROLL; u++) {
        const size_t i = base + (size_t)u * EW_THREADS;
        if (i < n_vec) {
#pragma unroll
            for (int k = 0; k < NIN; k++) r[u][k].load_stream(reinterpret_cast<const T *>(p.in[k]) + i * VEC);
        }
    }
#pragma unroll
    for (int u = 0; u < EW_UNROLL; u++) {
        const size_t i = base + (size_t)u * EW_THREADS;
        if (i < n_vec) {
            float fin[NIN][VEC], fout[NOUT][VEC];
#pragma unroll
            for (int k = 0; k < NIN; k++) r[u][k].unpack(fin[k]);
#pragma unroll
            for (int j = 0; j < VEC; j++) {
                float a[NIN], o[NOUT];
#pragma unroll
                for (int k = 0; k < NIN; k++) a[k] = fin[k][j];
                op(a, o);
#pragma unroll
                for (int k = 0; k < NOUT; k++) fout[k][j] = o[k];
            }
#pragma unroll
            for (int k = 0; k < NOUT; k++) {
                Raw<T, VEC> w;
                w.pack(fout[k]);
                w.store_stream(reinterpret_cast<T *>(p.out[k]) + i * VEC);
            }
        }
    }
    if (n_tail > 0 && blockIdx.x == 0 && threadIdx.x == 0) {
        for (int e = 0; e < n_tail; e++) {
            const size_t i = n_vec * VEC + e;
            float a[NIN], o[NOUT];
#pragma unroll
            for (int k = 0; k < NIN; k++) a[k] = Elt<T>::to_f(reinterpret_cast<const T *>(p.in[k])[i]);
            op(a, o);
#pragma unroll
            for (int k = 0; k < NOUT; k++) reinterpret_cast<T *>(p.out[k])[i] = Elt<T>::from_f(o[k]);
        }
    }
}

// Scalar body for pointers that are not 16-byte aligned.
template <typename T, int NIN, int NOUT, class Op>
__global__ void __launch_bounds__(EW_THREADS)
ew_scalar_kernel(EwPtrs<NIN, NOUT> p, size_t n, Op op) {
    for (size_t i = (size_t)blockIdx.x * EW_THREADS + threadIdx.x; i < n; i += (size_t)gridDim.x * EW_THREADS) {
        float a[NIN], o[NOUT];
#pragma unroll
        for (int k = 0; k < NIN; k++) a[k] = Elt<T>::to_f(reinterpret_cast<const T *>(p.in[k])[i]);
        op(a, o);
#pragma unroll
        for (int k = 0; k < NOUT; k++) reinterpret_cast<T *>(p.out[k])[i] = Elt<T>::from_f(o[k]);
    }
}

template <typename T, int NIN, int NOUT, class Op>
static int launch_ew(cudaStream_t st, const EwPtrs<NIN, NOUT> &p, size_t n, Op op) {
    bool al = true;
    for (int k = 0; k < NIN; k++) al = al && aligned16(p.in[k]);
    for (int k = 0; k < NOUT; k++) al = al && aligned16(p.out[k]);
    if (al) {
        constexpr int VEC = Elt<T>::VEC;
        const size_t n_vec = n / VEC;
        const int n_tail = (int)(n % VEC);
        size_t blocks = (n_vec + (size_t)EW_THREADS * EW_UNROLL - 1) / ((size_t)EW_THREADS * EW_UNROLL);
        if (blocks == 0) blocks = 1;
        if (blocks > 0x7fffffffull) return fail(ANE_CUDA_ERR_UNSUPPORTED, "element count %zu too large", n);
        launch_dep(DEP_EW, ew_vec_kernel<T, NIN, NOUT, Op>, dim3((unsigned)blocks), dim3(EW_THREADS), 0, st, p, n_vec, n_tail, op);
    } else {
        size_t blocks = (n + EW_THREADS - 1) / EW_THREADS;
        if (blocks > 148 * 32) blocks = 148 * 32;
        ew_scalar_kernel<T, NIN, NOUT, Op><<<(unsigned)blocks, EW_THREADS, 0, st>>>(p, n, op);
    }
    ANE_LAUNCH_OK(1);
    return ANE_CUDA_OK;
}

// ------------------------------------------------------------------ functors
// out = f*alpha + x                      training_dynamic/train.m:460 (vDSP_vsma), mil_dynamic.h:279-283
struct ResidualOp {
    float alpha;
    __device__ __forceinline__ void operator()(const float *a, float *o) const { o[0] = __fadd_rn(__fmul_rn(a[1], alpha), a[0]); }
};
// out = x*alpha                          train.m:497,523,595
struct ScaleOp {
    float alpha;
    __device__ __forceinline__ void operator()(const float *a, float *o) const { o[0] = a[0] * alpha; }
};
// sigmoid(x) = 1 / (1 + 2^(-x log2 e)) from the two hardware approximations (ex2.approx: 2 ulp, rcp.approx: 1 ulp): relative
// error below 1e-6, six instructions where expf and an IEEE division take about thirty.  Every operator runs at the
// board's power cap, so the instructions are paid for in bandwidth: measured over seconds of back-to-back launches the
// exact SwiGLU forward cost 174-178 pJ per byte where a plain copy costs 146 (5.7 against 6.8 TB/s); this form costs 142
// (7.0 TB/s), and the backward 144 instead of 159.  A sigmoid below the normal range (x < -87.3) comes out as zero.
__device__ __forceinline__ float sigmoid_fast(float x) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return r;
}
// out = (h1 / (1 + exp(-h1))) * h3       training/forward.h:101,149-151
struct SwigluOp {
    __device__ __forceinline__ void operator()(const float *a, float *o) const { o[0] = (a[0] * sigmoid_fast(a[0])) * a[1]; }
};
struct SwigluExactOp {            // knob "swiglu_exact": expf and IEEE division, the reference's expression literally
    __device__ __forceinline__ void operator()(const float *a, float *o) const {
        const float s = a[0] / (1.0f + expf(-a[0]));
        o[0] = s * a[1];
    }
};
// train.m:537-554: sig = 1/(1+exp(-h1)); dh3 = d*(h1*sig); dh1 = (d*h3)*(sig*(1 + h1*(1-sig)))
template <bool EXACT>
struct SwigluBwdOpT {
    __device__ __forceinline__ void operator()(const float *a, float *o) const {
        const float h1 = a[0], h3 = a[1], d = a[2];
        const float sig = EXACT ? 1.0f / (expf(-h1) + 1.0f) : sigmoid_fast(h1);
        o[1] = d * (h1 * sig);
        float t2 = -(sig + -1.0f);
        t2 = __fadd_rn(__fmul_rn(h1, t2), 1.0f);
        t2 = sig * t2;
        o[0] = (d * h3) * t2;
    }
};
struct SwigluBwdOp : SwigluBwdOpT<false> {};
struct SwigluBwdExactOp : SwigluBwdOpT<true> {};
// stories_cpu_ops.h:55-63 / training_dynamic/cpu_ops.h:56-64, same association order; the
// explicit _rn intrinsics keep the compiler from contracting the products into FMAs, so the
// result does not depend on how a CPU build of the same formula was compiled.
struct AdamOp {
    float b1, b2, omb1, omb2, bc1, bc2, lr, eps, wd, gscale;
    const float *clip;
    unsigned variant;
    bool use_gscale;
    __device__ __forceinline__ void operator()(const float *a, float *o) const {
        float w = a[0], g = a[1], m = a[2], v = a[3];
        if (use_gscale) g = __fmul_rn(g, gscale);
        if (clip) g = __fmul_rn(g, __ldg(clip));
        m = __fadd_rn(__fmul_rn(b1, m), __fmul_rn(omb1, g));
        v = __fadd_rn(__fmul_rn(b2, v), __fmul_rn(__fmul_rn(omb2, g), g));
        const float mh = __fdiv_rn(m, bc1), vh = __fdiv_rn(v, bc2);
        const float den = __fadd_rn(__fsqrt_rn(vh), eps);
        if (variant == ANE_ADAM_STORIES) {
            w = __fsub_rn(w, __fdiv_rn(__fmul_rn(lr, mh), den));
        } else {
            w = __fsub_rn(w, __fmul_rn(lr, __fadd_rn(__fdiv_rn(mh, den), __fmul_rn(wd, w))));
        }
        o[0] = w; o[1] = m; o[2] = v;
    }
};

// ------------------------------------------------------------------ gradient norm (two fixed-order stages)
constexpr int GN_THREADS = 256;
constexpr int GN_MAX_BLOCKS = 1184;  // 148 SMs x 8

__global__ void __launch_bounds__(GN_THREADS)
grad_norm_partial_kernel(const float *__restrict__ g, size_t n, float gscale, float *__restrict__ partial) {
    // Block b owns the contiguous chunk [b*chunk, (b+1)*chunk): the result does not depend on
    // scheduling, only on (n, gridDim).
    const size_t chunk = ((n + gridDim.x - 1) / gridDim.x + 3) & ~(size_t)3;
    const size_t lo = (size_t)blockIdx.x * chunk;
    const size_t hi = lo + chunk < n ? lo + chunk : n;
    float acc = 0.0f;
    if (lo < hi) {
        if ((reinterpret_cast<uintptr_t>(g) & 15u) == 0) {
            const size_t nv = (hi - lo) / 4;
            const float4 *gv = reinterpret_cast<const float4 *>(g + lo);
            for (size_t i = threadIdx.x; i < nv; i += GN_THREADS) {
                const float4 q = __ldcs(gv + i);
                const float a = q.x * gscale, b = q.y * gscale, c = q.z * gscale, d = q.w * gscale;
                acc += a * a; acc += b * b; acc += c * c; acc += d * d;
            }
            for (size_t i = lo + nv * 4 + threadIdx.x; i < hi; i += GN_THREADS) { const float a = g[i] * gscale; acc += a * a; }
        } else {
            for (size_t i = lo + threadIdx.x; i < hi; i += GN_THREADS) { const float a = g[i] * gscale; acc += a * a; }
        }
    }
    __shared__ float sh[GN_THREADS / 32];
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int i = 0; i < GN_THREADS / 32; i++) s += sh[i];
        partial[blockIdx.x] = s;
    }
}

__global__ void grad_norm_final_kernel(const float *__restrict__ partial, int nblocks, float *__restrict__ out) {
    // one warp, fixed order: lane l sums partial[l], partial[l+32], ...
    float acc = 0.0f;
    for (int i = threadIdx.x; i < nblocks; i += 32) acc += partial[i];
    acc = warp_sum(acc);
    if (threadIdx.x == 0) *out = acc;
}

// factor = clip/norm if clip > 0 and norm > clip else 1      train.m:788,809-810
__global__ void clip_factor_kernel(const float *__restrict__ normsq, int n_terms, float clip, float *__restrict__ factor) {
    float s = 0.0f;
    for (int i = 0; i < n_terms; i++) s += normsq[i];
    const float norm = sqrtf(s);
    *factor = (clip > 0.0f && norm > clip) ? clip / norm : 1.0f;
}

}  // namespace ane

using namespace ane;

extern "C" {

int ane_cuda_residual_dev(void *stream, ane_dtype dtype, size_t n, void *out, const void *x, const void *f, float alpha) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && x && f, "%s: null pointer", __func__);
    if (n == 0) return ANE_CUDA_OK;
    ANE_CHECK_EXTENT(out, n * dtype_size(dtype)); ANE_CHECK_EXTENT(x, n * dtype_size(dtype)); ANE_CHECK_EXTENT(f, n * dtype_size(dtype));
    EwPtrs<2, 1> p{{x, f}, {out}};
    ANE_DISPATCH_DTYPE(dtype, T, return (launch_ew<T, 2, 1>((cudaStream_t)stream, p, n, ResidualOp{alpha})));
    return ANE_CUDA_OK;
}

int ane_cuda_scale_dev(void *stream, ane_dtype dtype, size_t n, void *out, const void *x, float alpha) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && x, "%s: null pointer", __func__);
    if (n == 0) return ANE_CUDA_OK;
    ANE_CHECK_EXTENT(out, n * dtype_size(dtype)); ANE_CHECK_EXTENT(x, n * dtype_size(dtype));
    EwPtrs<1, 1> p{{x}, {out}};
    ANE_DISPATCH_DTYPE(dtype, T, return (launch_ew<T, 1, 1>((cudaStream_t)stream, p, n, ScaleOp{alpha})));
    return ANE_CUDA_OK;
}

int ane_cuda_swiglu_dev(void *stream, ane_dtype dtype, size_t n, void *out, const void *h1, const void *h3) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && h1 && h3, "%s: null pointer", __func__);
    if (n == 0) return ANE_CUDA_OK;
    ANE_CHECK_EXTENT(out, n * dtype_size(dtype)); ANE_CHECK_EXTENT(h1, n * dtype_size(dtype)); ANE_CHECK_EXTENT(h3, n * dtype_size(dtype));
    EwPtrs<2, 1> p{{h1, h3}, {out}};
    if (tuning("swiglu_exact", 0)) { ANE_DISPATCH_DTYPE(dtype, T, return (launch_ew<T, 2, 1>((cudaStream_t)stream, p, n, SwigluExactOp{}))); }
    ANE_DISPATCH_DTYPE(dtype, T, return (launch_ew<T, 2, 1>((cudaStream_t)stream, p, n, SwigluOp{})));
    return ANE_CUDA_OK;
}

int ane_cuda_swiglu_bwd_dev(void *stream, ane_dtype dtype, size_t n, void *dh1, void *dh3, const void *h1,
                            const void *h3, const void *dsilu) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dh1 && dh3 && h1 && h3 && dsilu, "%s: null pointer", __func__);
    if (n == 0) return ANE_CUDA_OK;
    ANE_CHECK_EXTENT(dh1, n * dtype_size(dtype)); ANE_CHECK_EXTENT(dh3, n * dtype_size(dtype)); ANE_CHECK_EXTENT(h1, n * dtype_size(dtype));
    ANE_CHECK_EXTENT(h3, n * dtype_size(dtype)); ANE_CHECK_EXTENT(dsilu, n * dtype_size(dtype));
    EwPtrs<3, 2> p{{h1, h3, dsilu}, {dh1, dh3}};
    if (tuning("swiglu_exact", 0)) { ANE_DISPATCH_DTYPE(dtype, T, return (launch_ew<T, 3, 2>((cudaStream_t)stream, p, n, SwigluBwdExactOp{}))); }
    ANE_DISPATCH_DTYPE(dtype, T, return (launch_ew<T, 3, 2>((cudaStream_t)stream, p, n, SwigluBwdOp{})));
    return ANE_CUDA_OK;
}

int ane_cuda_adam_dev(void *stream, size_t n, float *w, const float *g, float *m, float *v, int t, float lr,
                      float b1, float b2, float eps, float wd, float gscale, const float *clip_dev, unsigned flags) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(w && g && m && v, "%s: null pointer", __func__);
    ANE_REQUIRE(t >= 1, "%s: step t must be >= 1 (got %d)", __func__, t);
    ANE_REQUIRE(flags == ANE_ADAM_STORIES || flags == ANE_ADAM_DYNAMIC, "%s: bad flags %u", __func__, flags);
    if (n == 0) return ANE_CUDA_OK;
    ANE_CHECK_EXTENT(w, n * 4); ANE_CHECK_EXTENT(g, n * 4); ANE_CHECK_EXTENT(m, n * 4); ANE_CHECK_EXTENT(v, n * 4);
    AdamOp op;
    op.b1 = b1; op.b2 = b2;
    op.omb1 = 1 - b1; op.omb2 = 1 - b2;
    // bias corrections on the host with the host libm, as the reference computes them
    op.bc1 = 1.0f - powf(b1, t);
    op.bc2 = 1.0f - powf(b2, t);
    op.lr = lr; op.eps = eps; op.wd = wd; op.gscale = gscale;
    op.use_gscale = gscale != 1.0f;
    op.clip = clip_dev;
    op.variant = flags;
    EwPtrs<4, 3> p{{w, g, m, v}, {w, m, v}};
    return launch_ew<float, 4, 3>((cudaStream_t)stream, p, n, op);
}

int ane_cuda_grad_norm_sq_dev(void *stream, size_t n, const float *g, float gscale, float *out_dev) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(g && out_dev, "%s: null pointer", __func__);
    size_t blocks = (n + (size_t)GN_THREADS * 16 - 1) / ((size_t)GN_THREADS * 16);
    if (blocks < 1) blocks = 1;
    if (blocks > GN_MAX_BLOCKS) blocks = GN_MAX_BLOCKS;
    float *partial = static_cast<float *>(workspace(GN_MAX_BLOCKS * sizeof(float)));
    if (!partial) return fail(ANE_CUDA_ERR_NOMEM, "%s: no scratch", __func__);
    cudaStream_t st = (cudaStream_t)stream;
    grad_norm_partial_kernel<<<(unsigned)blocks, GN_THREADS, 0, st>>>(g, n, gscale, partial);
    grad_norm_final_kernel<<<1, 32, 0, st>>>(partial, (int)blocks, out_dev);
    ANE_LAUNCH_OK(2);
    return ANE_CUDA_OK;
}

int ane_cuda_clip_factor_dev(void *stream, const float *normsq_dev, int n_terms, float clip, float *factor_dev) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(normsq_dev && factor_dev && n_terms >= 1, "%s: bad argument", __func__);
    clip_factor_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(normsq_dev, n_terms, clip, factor_dev);
    ANE_LAUNCH_OK(1);
    return ANE_CUDA_OK;
}

}  // extern "C"
