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
// Returns a device scratch range of at least `bytes` (256-byte aligned) or nullptr.
void *workspace(size_t bytes);

#define ANE_REQUIRE_INIT() do { if (!::ane::ctx().inited) return ::ane::fail(ANE_CUDA_ERR_NOT_INIT, "%s: call ane_cuda_init first", __func__); } while (0)
#define ANE_REQUIRE(cond, ...) do { if (!(cond)) return ::ane::fail(ANE_CUDA_ERR_INVALID, __VA_ARGS__); } while (0)
#define ANE_CUDA_TRY(expr) do { cudaError_t e__ = (expr); if (e__ != cudaSuccess) return ::ane::fail(ANE_CUDA_ERR_CUDA, "%s: %s failed: %s", __func__, #expr, cudaGetErrorString(e__)); } while (0)
#define ANE_LAUNCH_OK(n) do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) return ::ane::fail(ANE_CUDA_ERR_CUDA, "%s: kernel launch failed: %s", __func__, cudaGetErrorString(e__)); ::ane::note_launch(n); } while (0)

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
};

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
