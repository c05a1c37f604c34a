// common.cuh -- shared device helpers and host plumbing for libane_cuda (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>

#include "../../include/ane_cuda.h"

namespace ane {

// ------------------------------------------------------------------ host plumbing
struct Context {
    bool inited = false;
    int device = -1;
    int sm_count = 0;
    void *ws = nullptr;            // grow-only scratch on the device
    size_t ws_bytes = 0;
    ane_cuda_status *status = nullptr;  // device status words
    void *pinned = nullptr;        // grow-only pinned staging for the host-pointer drop-ins
    size_t pinned_bytes = 0;
    void *stage = nullptr;         // grow-only device staging for the host-pointer drop-ins
    size_t stage_bytes = 0;
};
Context &ctx();
int fail(int code, const char *fmt, ...);
void note_launch(int n = 1);
// Returns a device scratch range of at least `bytes` (256-byte aligned) or nullptr.  A range that was handed out is never
// freed or moved before ane_cuda_shutdown: when the scratch has to grow, a new range is allocated and the old one is kept
// (a captured CUDA graph may hold its address).  After ane_cuda_freeze(1) a request that would grow fails instead.
void *workspace(size_t bytes);
// cudaMalloc behind the library's allocation-failure hook (tuning knob "fail_alloc" = number of coming allocations that
// fail as if the device were out of memory; host-side fault injection for the error paths).
cudaError_t dev_malloc(void **p, size_t bytes);
// Keeps a device range alive until ane_cuda_shutdown (ranges that were replaced but may still be referenced).
void retire_device_range(void *p);
bool frozen();
// Debug mode (tuning knob "check_extents" = 1, e.g. ANE_CUDA_TUNING=check_extents=1): before an operator is launched,
// every device range it is about to touch is checked against the allocation that holds the pointer (the driver knows the
// extent of every allocation).  A buffer that is too small for the given shape comes back as ANE_CUDA_ERR_INVALID with the
// argument's name instead of a stray write.  Off by default: one driver call per pointer.
int check_extent(const char *fn, const char *what, const void *p, size_t bytes);
bool check_extents_on();
#define ANE_CHECK_EXTENT(ptr, bytes)                                                                                      \
    do {                                                                                                                  \
        if (::ane::check_extents_on() && (ptr))                                                                           \
            if (int rc__ = ::ane::check_extent(__func__, #ptr, (ptr), (bytes))) return rc__;                              \
    } while (0)
// Kernel-selection knobs (ane_cuda_set_tuning); `dflt` when the knob was never set.
int tuning(const char *name, int dflt);
// Frees the cached RoPE cos/sin tables (rope.cu).
void rope_tables_release();
// Destroys the side stream and events of the embedding scatter-add (embed.cu).
void embed_side_release();
// Destroys the side stream and events of the Q / K pair operators (rope.cu).
void qk_side_release();

#define ANE_REQUIRE_INIT() do { if (!::ane::ctx().inited) return ::ane::fail(ANE_CUDA_ERR_NOT_INIT, "%s: call ane_cuda_init first", __func__); } while (0)
#define ANE_REQUIRE(cond, ...) do { if (!(cond)) return ::ane::fail(ANE_CUDA_ERR_INVALID, __VA_ARGS__); } while (0)
#define ANE_CUDA_TRY(expr) do { cudaError_t e__ = (expr); if (e__ != cudaSuccess) return ::ane::fail(ANE_CUDA_ERR_CUDA, "%s: %s failed: %s", __func__, #expr, cudaGetErrorString(e__)); } while (0)
#define ANE_LAUNCH_OK(n) do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) return ::ane::fail(ANE_CUDA_ERR_CUDA, "%s: kernel launch failed: %s", __func__, cudaGetErrorString(e__)); ::ane::note_launch(n); } while (0)

// Programmatic dependent launch (knob "dep_launch": a mask of kernel classes, default 0 = plain launches).  A kernel started
// through launch_dep() with its class enabled may be placed on the SMs while the kernel before it on the stream is still
// draining its last blocks: its blocks run their own set-up (index arithmetic, barrier initialisation) and then stop in
// dep_sync() until that kernel has completed and its memory is visible.  Rule for every kernel launched this way: NO access
// to global memory before dep_sync(), and every thread calls it.  dep_sync() then lets the kernel after this one be placed in
// turn.  Launched the plain way both instructions do nothing.
// Measured on B200 (benchmark step, 64-sequence micro-batches, ms per step): plain 299.2; element-wise kernels only 299.6;
// forward norms 300.1; column sums 299.2; QK ring kernels 298.9; cluster norm backward 309.7; everything 329.9 (SM clock at
// its maximum: the GPU idles); at 32 sequences 42.8-42.9 plain against 43.0-44.0.  Inside a graph the gaps between kernels
// are already short, and a persistent kernel whose grid is sized for an empty GPU is placed badly while blocks of the kernel
// before it still hold SMs (a cluster of four needs four free SMs of one GPC at the same time).  Hence off by default.
__device__ __forceinline__ void dep_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

enum DepClass { DEP_EW = 1, DEP_NORM_FWD = 2, DEP_NORM_BWD = 4, DEP_COLSUM = 8, DEP_QK = 16 };   // bits of knob "dep_launch"
#ifndef ANE_DEP_LAUNCH_DEFAULT
#define ANE_DEP_LAUNCH_DEFAULT 0
#endif

template <typename... KArgs, typename... Args>
static inline void launch_dep(int cls, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = (tuning("dep_launch", ANE_DEP_LAUNCH_DEFAULT) & cls) != 0 ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);      // the error, if any, is picked up by ANE_LAUNCH_OK
}

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline size_t dtype_size(ane_dtype d) { return d == ANE_F32 ? 4 : 2; }
static inline bool dtype_ok(ane_dtype d) { return d == ANE_F32 || d == ANE_BF16 || d == ANE_F16; }
static inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Dispatch a templated launcher on the activation dtype.
#define ANE_DISPATCH_DTYPE(dtype, T, ...)                                   \
    switch (dtype) {                                                        \
        case ANE_F32:  { using T = float;          __VA_ARGS__; } break;    \
        case ANE_BF16: { using T = __nv_bfloat16;  __VA_ARGS__; } break;    \
        case ANE_F16:  { using T = __half;         __VA_ARGS__; } break;    \
        default: return ::ane::fail(ANE_CUDA_ERR_INVALID, "%s: bad dtype %d", __func__, (int)dtype); \
    }

// ------------------------------------------------------------------ device helpers
#ifdef __CUDACC__

template <typename T> struct Elt;
template <> struct Elt<float> {
    static constexpr int VEC = 4;
    __device__ __forceinline__ static float to_f(float v) { return v; }
    __device__ __forceinline__ static float from_f(float v) { return v; }
    __device__ __forceinline__ static void unpack(const uint4 &r, float *f) {
        f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y);
        f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
    }
    __device__ __forceinline__ static uint4 pack(const float *f) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
    __device__ __forceinline__ static void unpack2(const uint4 &r, float2 *p) {
        p[0] = make_float2(__uint_as_float(r.x), __uint_as_float(r.y));
        p[1] = make_float2(__uint_as_float(r.z), __uint_as_float(r.w));
    }
    __device__ __forceinline__ static uint4 pack2(const float2 *p) {
        return make_uint4(__float_as_uint(p[0].x), __float_as_uint(p[0].y), __float_as_uint(p[1].x), __float_as_uint(p[1].y));
    }
};
template <> struct Elt<__nv_bfloat16> {
    static constexpr int VEC = 8;
    __device__ __forceinline__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ __forceinline__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
    __device__ __forceinline__ static void unpack(const uint4 &r, float *f) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ __forceinline__ static uint4 pack(const float *f) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&p);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ __forceinline__ static void unpack2(const uint4 &r, float2 *p) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; i++) p[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
    }
    __device__ __forceinline__ static uint4 pack2(const float2 *p) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            __nv_bfloat162 q = __floats2bfloat162_rn(p[i].x, p[i].y);
            w[i] = *reinterpret_cast<uint32_t *>(&q);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <> struct Elt<__half> {
    static constexpr int VEC = 8;
    __device__ __forceinline__ static float to_f(__half v) { return __half2float(v); }
    __device__ __forceinline__ static __half from_f(float v) { return __float2half_rn(v); }
    __device__ __forceinline__ static void unpack(const uint4 &r, float *f) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            __half2 h = *reinterpret_cast<const __half2 *>(&w[i]);
            float2 v = __half22float2(h);
            f[2 * i] = v.x; f[2 * i + 1] = v.y;
        }
    }
    __device__ __forceinline__ static uint4 pack(const float *f) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            __half2 p = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&p);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ __forceinline__ static void unpack2(const uint4 &r, float2 *p) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; i++) p[i] = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
    }
    __device__ __forceinline__ static uint4 pack2(const float2 *p) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            __half2 q = __floats2half2_rn(p[i].x, p[i].y);
            w[i] = *reinterpret_cast<uint32_t *>(&q);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// ------------------------------------------------------------------ packed fp32 lanes
// Blackwell issues two fp32 operations per instruction on register pairs (add/sub/mul/fma
// .f32x2).  The reduction kernels are close to issue-bound in bf16 (about 20 B of HBM traffic per
// SM and clock against 4 issue slots), so their per-element math runs on V<N>: N fp32 lanes
// held as N/2 pairs.  Every packed operation rounds each lane exactly like the scalar IEEE
// operation, so results do not depend on the packing.
__device__ __forceinline__ float2 f2_fma(float2 a, float2 b, float2 c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(*reinterpret_cast<unsigned long long *>(&a)),
        "l"(*reinterpret_cast<unsigned long long *>(&b)), "l"(*reinterpret_cast<unsigned long long *>(&c)));
    return *reinterpret_cast<float2 *>(&d);
}
__device__ __forceinline__ float2 f2_mul(float2 a, float2 b) {
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<unsigned long long *>(&a)),
        "l"(*reinterpret_cast<unsigned long long *>(&b)));
    return *reinterpret_cast<float2 *>(&d);
}
__device__ __forceinline__ float2 f2_add(float2 a, float2 b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<unsigned long long *>(&a)),
        "l"(*reinterpret_cast<unsigned long long *>(&b)));
    return *reinterpret_cast<float2 *>(&d);
}
__device__ __forceinline__ float2 f2_sub(float2 a, float2 b) {
    unsigned long long d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<unsigned long long *>(&a)),
        "l"(*reinterpret_cast<unsigned long long *>(&b)));
    return *reinterpret_cast<float2 *>(&d);
}

template <int N> struct V {
    static_assert(N % 2 == 0, "V<N> holds pairs");
    float2 p[N / 2];
    __device__ __forceinline__ static V splat(float s) {
        V r;
#pragma unroll
        for (int i = 0; i < N / 2; i++) r.p[i] = make_float2(s, s);
        return r;
    }
    __device__ __forceinline__ float get(int j) const { return (j & 1) ? p[j >> 1].y : p[j >> 1].x; }
    __device__ __forceinline__ void set(int j, float v) { if (j & 1) p[j >> 1].y = v; else p[j >> 1].x = v; }
    // Sum of the N lanes in a fixed tree order: packed adds halve the pair count each step, the last pair is added
    // across.  (N / 2 must be a power of two: 2, 4 or 8 lanes in every use.)
    __device__ __forceinline__ float hsum() const {
        float2 t[N / 2];
#pragma unroll
        for (int i = 0; i < N / 2; i++) t[i] = p[i];
#pragma unroll
        for (int w = N / 4; w >= 1; w >>= 1) {
#pragma unroll
            for (int i = 0; i < w; i++) t[i] = f2_add(t[i], t[i + w]);
        }
        return t[0].x + t[0].y;
    }
};
template <> struct V<1> {
    float a;
    __device__ __forceinline__ static V splat(float s) { V r; r.a = s; return r; }
    __device__ __forceinline__ float get(int) const { return a; }
    __device__ __forceinline__ void set(int, float v) { a = v; }
    __device__ __forceinline__ float hsum() const { return a; }
};
template <int N> __device__ __forceinline__ V<N> vmul(const V<N> &a, const V<N> &b) {
    V<N> r;
#pragma unroll
    for (int i = 0; i < N / 2; i++) r.p[i] = f2_mul(a.p[i], b.p[i]);
    return r;
}
template <int N> __device__ __forceinline__ V<N> vadd(const V<N> &a, const V<N> &b) {
    V<N> r;
#pragma unroll
    for (int i = 0; i < N / 2; i++) r.p[i] = f2_add(a.p[i], b.p[i]);
    return r;
}
template <int N> __device__ __forceinline__ V<N> vsub(const V<N> &a, const V<N> &b) {
    V<N> r;
#pragma unroll
    for (int i = 0; i < N / 2; i++) r.p[i] = f2_sub(a.p[i], b.p[i]);
    return r;
}
template <int N> __device__ __forceinline__ V<N> vfma(const V<N> &a, const V<N> &b, const V<N> &c) {
    V<N> r;
#pragma unroll
    for (int i = 0; i < N / 2; i++) r.p[i] = f2_fma(a.p[i], b.p[i], c.p[i]);
    return r;
}
// a * (s, s): the per-channel weight lives in one register pair, not in N lanes
template <int N> __device__ __forceinline__ V<N> vscale(const V<N> &a, float s) {
    V<N> r;
    const float2 s2 = make_float2(s, s);
#pragma unroll
    for (int i = 0; i < N / 2; i++) r.p[i] = f2_mul(a.p[i], s2);
    return r;
}
template <int N> __device__ __forceinline__ V<N> vfma_s(const V<N> &a, float s, const V<N> &c) {
    V<N> r;
    const float2 s2 = make_float2(s, s);
#pragma unroll
    for (int i = 0; i < N / 2; i++) r.p[i] = f2_fma(a.p[i], s2, c.p[i]);
    return r;
}
template <> __device__ __forceinline__ V<1> vscale<1>(const V<1> &a, float s) { V<1> r; r.a = __fmul_rn(a.a, s); return r; }
template <> __device__ __forceinline__ V<1> vfma_s<1>(const V<1> &a, float s, const V<1> &c) { V<1> r; r.a = fmaf(a.a, s, c.a); return r; }
template <> __device__ __forceinline__ V<1> vmul<1>(const V<1> &a, const V<1> &b) { V<1> r; r.a = __fmul_rn(a.a, b.a); return r; }
template <> __device__ __forceinline__ V<1> vadd<1>(const V<1> &a, const V<1> &b) { V<1> r; r.a = __fadd_rn(a.a, b.a); return r; }
template <> __device__ __forceinline__ V<1> vsub<1>(const V<1> &a, const V<1> &b) { V<1> r; r.a = __fsub_rn(a.a, b.a); return r; }
template <> __device__ __forceinline__ V<1> vfma<1>(const V<1> &a, const V<1> &b, const V<1> &c) { V<1> r; r.a = fmaf(a.a, b.a, c.a); return r; }

// Shared-memory transfer of the N lanes of a V<N> as 16-byte words: a quarter-warp of such
// stores covers one contiguous run, so rows of per-token partials are written without bank
// conflicts (scalar stores of lane j from 8 lanes x 4 row groups would collide 8 ways).
template <int N> __device__ __forceinline__ void lanes_to_smem(float *dst, const V<N> &v) {
#pragma unroll
    for (int i = 0; i < N / 4; i++)
        *reinterpret_cast<float4 *>(dst + 4 * i) = make_float4(v.p[2 * i].x, v.p[2 * i].y, v.p[2 * i + 1].x, v.p[2 * i + 1].y);
}
template <> __device__ __forceinline__ void lanes_to_smem<1>(float *dst, const V<1> &v) { dst[0] = v.a; }
template <int N> __device__ __forceinline__ V<N> lanes_from_smem(const float *src) {
    V<N> v;
#pragma unroll
    for (int i = 0; i < N / 4; i++) {
        const float4 q = *reinterpret_cast<const float4 *>(src + 4 * i);
        v.p[2 * i] = make_float2(q.x, q.y);
        v.p[2 * i + 1] = make_float2(q.z, q.w);
    }
    return v;
}
template <> __device__ __forceinline__ V<1> lanes_from_smem<1>(const float *src) { V<1> v; v.a = src[0]; return v; }

// Column sums of a shared-memory matrix red[R][COLS] with ALL `THREADS` threads of the block
// (THREADS == COLS * P): thread tid adds R/P rows of column tid / P, the P partial sums meet
// through warp shuffles, and every thread of the group returns the column total.  Compared with
// one thread per column this shortens the serial chain from R to R/P loads while the rest of the
// block would only wait at the next barrier.  The summation order is fixed.
template <int R, int COLS, int THREADS>
__device__ __forceinline__ float block_column_sum(const float *red, int tid) {
    constexpr int P = THREADS / COLS;
    static_assert(P >= 1 && P <= 32 && (P & (P - 1)) == 0 && COLS * P == THREADS && R % P == 0, "bad reduction shape");
    const int col = tid / P, part = tid % P;
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < R / P; i++) s += red[(part * (R / P) + i) * COLS + col];
#pragma unroll
    for (int off = P / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    return s;
}

// lane-wise sum over the row groups of a warp (lanes with equal lane % LG), every lane gets the total
template <int N, int LG>
__device__ __forceinline__ V<N> warp_rowgroup_sum(V<N> v) {
#pragma unroll
    for (int off = LG; off < 32; off <<= 1) {
#pragma unroll
        for (int i = 0; i < N / 2; i++) {
            v.p[i].x += __shfl_xor_sync(0xffffffffu, v.p[i].x, off);
            v.p[i].y += __shfl_xor_sync(0xffffffffu, v.p[i].y, off);
        }
    }
    return v;
}

// out[c] += sum over rows r of partial[r][c], in a fixed order: 32 columns x 8 row slices per block, every thread
// walks its slice with eight independent loads in flight, the slices are added in slice order.  (One thread per
// column walking all rows took 19 us for 444 x 1024 partials: a chain of dependent-latency loads.)
template <int UNUSED = 0>
__global__ void __launch_bounds__(256) column_sum_add_kernel(float *__restrict__ out, const float *__restrict__ partial, int rows, int cols) {
    __shared__ float acc[8][32];
    const int cl = threadIdx.x & 31, sl = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + cl;
    const int per = (rows + 7) / 8;
    const int r0 = sl * per, r1 = r0 + per < rows ? r0 + per : rows;
    float s = 0.0f;
    dep_sync();
    if (c < cols) {
        int r = r0;
        for (; r + 8 <= r1; r += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; u++) v[u] = partial[(size_t)(r + u) * cols + c];
#pragma unroll
            for (int u = 0; u < 8; u++) s += v[u];
        }
        for (; r < r1; r++) s += partial[(size_t)r * cols + c];
    }
    acc[sl][cl] = s;
    __syncthreads();
    if (sl == 0 && c < cols) {
        float t = 0.0f;
#pragma unroll
        for (int q = 0; q < 8; q++) t += acc[q][cl];
        out[c] += t;
    }
}

// A group of VEC consecutive elements held raw: one 16-byte word when VEC is the full vector
// width of T, one element when VEC == 1 (the path for shapes that break 16-byte alignment).
template <typename T, int VEC> struct Raw;
template <typename T> struct Raw<T, 1> {
    T v;
    __device__ __forceinline__ void load(const T *p) { v = *p; }
    __device__ __forceinline__ void load_stream(const T *p) { v = __ldcs(p); }
    __device__ __forceinline__ void store(T *p) const { *p = v; }
    __device__ __forceinline__ void store_stream(T *p) const { __stcs(p, v); }
    __device__ __forceinline__ void unpack(float *f) const { f[0] = Elt<T>::to_f(v); }
    __device__ __forceinline__ void pack(const float *f) { v = Elt<T>::from_f(f[0]); }
    __device__ __forceinline__ V<1> get() const { V<1> r; r.a = Elt<T>::to_f(v); return r; }
    __device__ __forceinline__ void put(const V<1> &x) { v = Elt<T>::from_f(x.a); }
};
#define ANE_RAW_FULL(T)                                                                                   \
    template <> struct Raw<T, Elt<T>::VEC> {                                                              \
        uint4 v;                                                                                          \
        __device__ __forceinline__ void load(const T *p) { v = *reinterpret_cast<const uint4 *>(p); }     \
        __device__ __forceinline__ void load_stream(const T *p) { v = __ldcs(reinterpret_cast<const uint4 *>(p)); } \
        __device__ __forceinline__ void store(T *p) const { *reinterpret_cast<uint4 *>(p) = v; }          \
        __device__ __forceinline__ void store_stream(T *p) const { __stcs(reinterpret_cast<uint4 *>(p), v); } \
        __device__ __forceinline__ void unpack(float *f) const { Elt<T>::unpack(v, f); }                  \
        __device__ __forceinline__ void pack(const float *f) { v = Elt<T>::pack(f); }                     \
        __device__ __forceinline__ V<Elt<T>::VEC> get() const { V<Elt<T>::VEC> r; Elt<T>::unpack2(v, r.p); return r; } \
        __device__ __forceinline__ void put(const V<Elt<T>::VEC> &x) { v = Elt<T>::pack2(x.p); }          \
    };
ANE_RAW_FULL(float)
ANE_RAW_FULL(__nv_bfloat16)
ANE_RAW_FULL(__half)
#undef ANE_RAW_FULL

// Round an fp32 value through the storage type (what a separate kernel reading the stored
// tensor would see).
template <typename T> __device__ __forceinline__ float round_through(float v) { return Elt<T>::to_f(Elt<T>::from_f(v)); }
template <> __device__ __forceinline__ float round_through<float>(float v) { return v; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

#endif  // __CUDACC__

// RoPE inverse frequencies, computed on the host exactly as the reference does
// (freq = 1/powf(base, 2*i/hd), training_dynamic/cpu_ops.h:172) and handed to the kernels by
// value: theta = p*freq is ill-conditioned in fp32 (one ulp of freq moves theta by up to 1e-4
// at p = 2047), so the table must carry the host libm's bits, not the device powf's.
struct RopeFreq { float f[128]; };   // hd <= 256

}  // namespace ane
