// layout.cu -- the data-movement helpers that sit on either side of the operator set in the reference's
// training loop: GQA head tiling / head-sum (training_dynamic/io.h:327-351), fp32 <-> 16-bit conversion and
// the "activations + weights on one spatial axis" packing (stories_io.h:41-84, training_dynamic/io.h:79-96),
// vocabulary compaction (training_dynamic/cpu_ops.h:96-148).  All of it is streaming or row-gather work.
#include "common.cuh"

#include <cub/device/device_scan.cuh>

namespace ane {

constexpr int LY_THREADS = 256;

// ------------------------------------------------------------------ GQA tile / reduce
// x: [B][heads*HD][S].  One "head block" is HD*S contiguous elements; hb_vec = vectors per head block.
// tile:   out[b][kv*ratio + r] = in[b][kv]            (io.h:330-337: a memcpy per query head)
// A thread reads one input vector and writes it `ratio` times: the input crosses HBM once.
template <int VECB>
__global__ void __launch_bounds__(LY_THREADS)
gqa_tile_kernel(char *__restrict__ out, const char *__restrict__ in, size_t hb_units, int kv_heads, int ratio, int B) {
    const size_t total = (size_t)B * kv_heads * hb_units;
    for (size_t i = (size_t)blockIdx.x * LY_THREADS + threadIdx.x; i < total; i += (size_t)gridDim.x * LY_THREADS) {
        const size_t head = i / hb_units, off = i - head * hb_units;          // head = b*kv_heads + kv
        if (VECB == 16) {
            const uint4 v = __ldcs(reinterpret_cast<const uint4 *>(in) + i);
            for (int r = 0; r < ratio; r++) __stcs(reinterpret_cast<uint4 *>(out) + (head * ratio + r) * hb_units + off, v);
        } else if (VECB == 4) {
            const uint32_t v = reinterpret_cast<const uint32_t *>(in)[i];
            for (int r = 0; r < ratio; r++) reinterpret_cast<uint32_t *>(out)[(head * ratio + r) * hb_units + off] = v;
        } else {
            const uint16_t v = reinterpret_cast<const uint16_t *>(in)[i];
            for (int r = 0; r < ratio; r++) reinterpret_cast<uint16_t *>(out)[(head * ratio + r) * hb_units + off] = v;
        }
    }
}

// reduce: out[b][kv] = ((0 + in[b][kv*ratio]) + in[b][kv*ratio+1]) + ...   (io.h:340-351: memset, then += per head)
template <typename T, int VEC>
__global__ void __launch_bounds__(LY_THREADS)
gqa_reduce_kernel(T *__restrict__ out, const T *__restrict__ in, size_t hb_vec, int kv_heads, int ratio, int B) {
    const size_t total = (size_t)B * kv_heads * hb_vec;
    for (size_t i = (size_t)blockIdx.x * LY_THREADS + threadIdx.x; i < total; i += (size_t)gridDim.x * LY_THREADS) {
        const size_t head = i / hb_vec, off = i - head * hb_vec;
        float acc[VEC];
#pragma unroll
        for (int j = 0; j < VEC; j++) acc[j] = 0.0f;
        for (int r0 = 0; r0 < ratio; r0 += 4) {          // four heads in flight; added in head order
            Raw<T, VEC> v[4];
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (r0 + u < ratio) v[u].load_stream(in + ((head * ratio + r0 + u) * hb_vec + off) * VEC);
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (r0 + u < ratio) {
                    float f[VEC];
                    v[u].unpack(f);
#pragma unroll
                    for (int j = 0; j < VEC; j++) acc[j] = __fadd_rn(acc[j], f[j]);
                }
        }
        Raw<T, VEC> o;
        o.pack(acc);
        o.store_stream(out + i * VEC);
    }
}

// ------------------------------------------------------------------ conversion
// dst[i] = (TD)src[i], round to nearest even like the NEON vcvt the reference uses (stories_io.h:41-58).
template <typename TD, typename TS>
__global__ void __launch_bounds__(LY_THREADS)
convert_kernel(TD *__restrict__ dst, const TS *__restrict__ src, size_t n) {
    // eight elements per thread and step where both sides are 16-byte aligned for that
    const size_t n8 = n / 8;
    const bool al = (reinterpret_cast<uintptr_t>(dst) & 15u) == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
    const size_t gsz = (size_t)gridDim.x * LY_THREADS, tid = (size_t)blockIdx.x * LY_THREADS + threadIdx.x;
    if (al) {
        for (size_t i = tid; i < n8; i += gsz) {
            float f[8];
            if (sizeof(TS) == 4) {
                const float4 a = __ldcs(reinterpret_cast<const float4 *>(src) + 2 * i), b = __ldcs(reinterpret_cast<const float4 *>(src) + 2 * i + 1);
                f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
            } else {
                const uint4 a = __ldcs(reinterpret_cast<const uint4 *>(src) + i);
                const TS *h = reinterpret_cast<const TS *>(&a);
#pragma unroll
                for (int j = 0; j < 8; j++) f[j] = Elt<TS>::to_f(h[j]);
            }
            if (sizeof(TD) == 4) {
                __stcs(reinterpret_cast<float4 *>(dst) + 2 * i, make_float4(f[0], f[1], f[2], f[3]));
                __stcs(reinterpret_cast<float4 *>(dst) + 2 * i + 1, make_float4(f[4], f[5], f[6], f[7]));
            } else {
                uint4 o;
                TD *h = reinterpret_cast<TD *>(&o);
#pragma unroll
                for (int j = 0; j < 8; j++) h[j] = Elt<TD>::from_f(f[j]);
                __stcs(reinterpret_cast<uint4 *>(dst) + i, o);
            }
        }
        for (size_t i = n8 * 8 + tid; i < n; i += gsz) dst[i] = Elt<TD>::from_f(Elt<TS>::to_f(src[i]));
    } else {
        for (size_t i = tid; i < n; i += gsz) dst[i] = Elt<TD>::from_f(Elt<TS>::to_f(src[i]));
    }
}

// io_write_dyn (io.h:79-88): row d of the packed surface = [ act[d][0..seq) | W[d][0..oc) ] in 16-bit
template <typename TD>
__global__ void __launch_bounds__(LY_THREADS)
pack_dyn_kernel(TD *__restrict__ buf, const float *__restrict__ act, const float *__restrict__ W, int ic, int seq, int oc) {
    const int sp = seq + oc;
    const int d = blockIdx.y;
    for (int i = blockIdx.x * LY_THREADS + threadIdx.x; i < sp; i += gridDim.x * LY_THREADS) {
        const float v = i < seq ? __ldg(act + (size_t)d * seq + i) : __ldg(W + (size_t)d * oc + (i - seq));
        buf[(size_t)d * sp + i] = Elt<TD>::from_f(v);
    }
}

// ------------------------------------------------------------------ vocabulary compaction
__global__ void vocab_clear_kernel(int *__restrict__ flags, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) flags[i] = 0;
}
template <typename ID>
__global__ void vocab_mark_kernel(int *__restrict__ flags, const void *__restrict__ tokens, size_t n, int vocab, ane_cuda_status *status) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int id = (int)reinterpret_cast<const ID *>(tokens)[i];
        if (id >= 0 && id < vocab) flags[id] = 1;        // every writer stores 1
        else atomicAdd(&status->oor_ids, 1);
    }
}
// scan[v] = number of used ids below v  ->  full_to_compact, compact_to_full, count   (cpu_ops.h:112-126)
__global__ void vocab_assign_kernel(int *__restrict__ full_to_compact, int *__restrict__ compact_to_full, int *__restrict__ count,
                                    const int *__restrict__ flags, const int *__restrict__ scan, int vocab) {
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= vocab) return;
    const int used = flags[v], c = scan[v];
    full_to_compact[v] = used ? c : -1;
    if (used) compact_to_full[c] = v;
    if (v == vocab - 1) *count = c + used;
}

// Row movers, a warp per row of `dim` floats; map[c] = full-vocabulary row of compact row c.
//   MODE 0: compact[c] = full[map[c]]          vocab_compact_embed   cpu_ops.h:129-134
//   MODE 1: full[map[c]] += compact[c]         vocab_scatter_grads   cpu_ops.h:137-143
//   MODE 2: full[map[c]] = compact[c]          vocab_update_full     cpu_ops.h:146-149
template <int MODE>
__global__ void __launch_bounds__(LY_THREADS)
vocab_rows_kernel(float *__restrict__ full, float *__restrict__ compact, const int *__restrict__ map, const int *__restrict__ count_dev,
                  int count_max, int dim, int full_vocab) {
    const int lane = threadIdx.x & 31;
    const int nrows = count_dev ? min(*count_dev, count_max) : count_max;
    const bool v4 = (dim & 3) == 0 && (reinterpret_cast<uintptr_t>(full) & 15u) == 0 && (reinterpret_cast<uintptr_t>(compact) & 15u) == 0;
    for (int c = blockIdx.x * (LY_THREADS / 32) + (threadIdx.x >> 5); c < nrows; c += gridDim.x * (LY_THREADS / 32)) {
        const int fv = map[c];
        if (fv < 0 || fv >= full_vocab) continue;
        float *fr = full + (size_t)fv * dim, *cr = compact + (size_t)c * dim;
        if (v4) {
            for (int d = lane * 4; d < dim; d += 128) {
                float4 *fp = reinterpret_cast<float4 *>(fr + d), *cp = reinterpret_cast<float4 *>(cr + d);
                if (MODE == 0) *cp = *fp;
                else if (MODE == 2) *fp = *cp;
                else {
                    float4 a = *fp;
                    const float4 b = *cp;
                    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
                    *fp = a;
                }
            }
        } else {
            for (int d = lane; d < dim; d += 32) {
                if (MODE == 0) cr[d] = fr[d];
                else if (MODE == 2) fr[d] = cr[d];
                else fr[d] += cr[d];
            }
        }
    }
}

static unsigned flat_grid(size_t items) {
    size_t b = (items + LY_THREADS - 1) / LY_THREADS;
    const size_t cap = (size_t)ctx().sm_count * 16;
    if (b > cap) b = cap;
    return (unsigned)(b < 1 ? 1 : b);
}

}  // namespace ane

using namespace ane;

namespace {
template <typename T>
int launch_gqa_reduce(cudaStream_t st, int B, int kv_heads, int ratio, int hd, int S, void *out, const void *in) {
    constexpr int VEC = Elt<T>::VEC;
    const size_t hb = (size_t)hd * S;
    if (hb % VEC == 0 && aligned16(out) && aligned16(in)) {
        gqa_reduce_kernel<T, VEC><<<flat_grid((size_t)B * kv_heads * (hb / VEC)), LY_THREADS, 0, st>>>((T *)out, (const T *)in, hb / VEC, kv_heads, ratio, B);
    } else {
        gqa_reduce_kernel<T, 1><<<flat_grid((size_t)B * kv_heads * hb), LY_THREADS, 0, st>>>((T *)out, (const T *)in, hb, kv_heads, ratio, B);
    }
    ANE_LAUNCH_OK(1);
    return ANE_CUDA_OK;
}
}  // namespace

extern "C" {

int ane_cuda_gqa_tile_dev(void *stream, ane_dtype dtype, int B, int kv_heads, int ratio, int hd, int S, void *out, const void *in) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && in, "%s: null pointer", __func__);
    ANE_REQUIRE(dtype_ok(dtype), "%s: bad dtype", __func__);
    ANE_REQUIRE(B >= 1 && kv_heads >= 1 && ratio >= 1 && hd >= 1 && S >= 1, "%s: bad shape", __func__);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t esz = dtype_size(dtype);
    const size_t hb_bytes = (size_t)hd * S * esz;
    if (hb_bytes % 16 == 0 && aligned16(out) && aligned16(in)) {
        const size_t units = hb_bytes / 16;
        gqa_tile_kernel<16><<<flat_grid((size_t)B * kv_heads * units), LY_THREADS, 0, st>>>((char *)out, (const char *)in, units, kv_heads, ratio, B);
    } else if (esz == 4) {
        const size_t units = (size_t)hd * S;
        gqa_tile_kernel<4><<<flat_grid((size_t)B * kv_heads * units), LY_THREADS, 0, st>>>((char *)out, (const char *)in, units, kv_heads, ratio, B);
    } else {
        const size_t units = (size_t)hd * S;
        gqa_tile_kernel<2><<<flat_grid((size_t)B * kv_heads * units), LY_THREADS, 0, st>>>((char *)out, (const char *)in, units, kv_heads, ratio, B);
    }
    ANE_LAUNCH_OK(1);
    return ANE_CUDA_OK;
}


int ane_cuda_gqa_reduce_dev(void *stream, ane_dtype dtype, int B, int kv_heads, int ratio, int hd, int S, void *out, const void *in) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && in, "%s: null pointer", __func__);
    ANE_REQUIRE(dtype_ok(dtype), "%s: bad dtype", __func__);
    ANE_REQUIRE(B >= 1 && kv_heads >= 1 && ratio >= 1 && hd >= 1 && S >= 1, "%s: bad shape", __func__);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == ANE_F32) return launch_gqa_reduce<float>(st, B, kv_heads, ratio, hd, S, out, in);
    if (dtype == ANE_BF16) return launch_gqa_reduce<__nv_bfloat16>(st, B, kv_heads, ratio, hd, S, out, in);
    return launch_gqa_reduce<__half>(st, B, kv_heads, ratio, hd, S, out, in);
}

int ane_cuda_convert_dev(void *stream, ane_dtype dst_dtype, ane_dtype src_dtype, size_t n, void *dst, const void *src) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dst && src, "%s: null pointer", __func__);
    ANE_REQUIRE(dtype_ok(dst_dtype) && dtype_ok(src_dtype), "%s: bad dtype", __func__);
    if (n == 0) return ANE_CUDA_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = flat_grid((n + 7) / 8);
#define ANE_CVT(DE, TD, SE, TS) \
    if (dst_dtype == DE && src_dtype == SE) convert_kernel<TD, TS><<<grid, LY_THREADS, 0, st>>>((TD *)dst, (const TS *)src, n); else
    ANE_CVT(ANE_F16, __half, ANE_F32, float)
    ANE_CVT(ANE_BF16, __nv_bfloat16, ANE_F32, float)
    ANE_CVT(ANE_F32, float, ANE_F16, __half)
    ANE_CVT(ANE_F32, float, ANE_BF16, __nv_bfloat16)
    ANE_CVT(ANE_F16, __half, ANE_BF16, __nv_bfloat16)
    ANE_CVT(ANE_BF16, __nv_bfloat16, ANE_F16, __half)
    ANE_CVT(ANE_F32, float, ANE_F32, float)
    ANE_CVT(ANE_F16, __half, ANE_F16, __half)
    ANE_CVT(ANE_BF16, __nv_bfloat16, ANE_BF16, __nv_bfloat16)
    return fail(ANE_CUDA_ERR_INVALID, "%s: unsupported conversion", __func__);
#undef ANE_CVT
    ANE_LAUNCH_OK(1);
    return ANE_CUDA_OK;
}

int ane_cuda_pack_dyn_dev(void *stream, ane_dtype dst_dtype, int ic, int seq, int oc, void *buf, const float *act, const float *W) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(buf && act && W, "%s: null pointer", __func__);
    ANE_REQUIRE(dst_dtype == ANE_F16 || dst_dtype == ANE_BF16, "%s: the packed surface is 16-bit", __func__);
    ANE_REQUIRE(ic >= 1 && seq >= 1 && oc >= 1 && ic <= 65535, "%s: bad shape ic=%d seq=%d oc=%d", __func__, ic, seq, oc);
    cudaStream_t st = (cudaStream_t)stream;
    const int sp = seq + oc;
    dim3 grid((unsigned)((sp + LY_THREADS * 4 - 1) / (LY_THREADS * 4)), (unsigned)ic);
    if (dst_dtype == ANE_F16) pack_dyn_kernel<__half><<<grid, LY_THREADS, 0, st>>>((__half *)buf, act, W, ic, seq, oc);
    else pack_dyn_kernel<__nv_bfloat16><<<grid, LY_THREADS, 0, st>>>((__nv_bfloat16 *)buf, act, W, ic, seq, oc);
    ANE_LAUNCH_OK(1);
    return ANE_CUDA_OK;
}

int ane_cuda_vocab_map_build_dev(void *stream, ane_idtype idtype, size_t n_tokens, const void *tokens, int full_vocab,
                                 int *full_to_compact, int *compact_to_full, int *compact_vocab) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(tokens && full_to_compact && compact_to_full && compact_vocab, "%s: null pointer", __func__);
    ANE_REQUIRE(idtype == ANE_ID_U16 || idtype == ANE_ID_I32, "%s: bad id type", __func__);
    ANE_REQUIRE(full_vocab >= 1 && n_tokens >= 1, "%s: bad sizes", __func__);
    cudaStream_t st = (cudaStream_t)stream;
    size_t cub_bytes = 0;
    ANE_CUDA_TRY(cub::DeviceScan::ExclusiveSum(nullptr, cub_bytes, (const int *)nullptr, (int *)nullptr, full_vocab, st));
    const size_t ints = round_up((size_t)full_vocab * sizeof(int), 256);
    char *ws = static_cast<char *>(workspace(2 * ints + round_up(cub_bytes, 256)));
    if (!ws) return fail(ANE_CUDA_ERR_NOMEM, "%s: no scratch", __func__);
    int *flags = (int *)ws, *scan = (int *)(ws + ints);
    const int vb = (full_vocab + 255) / 256;
    vocab_clear_kernel<<<vb, 256, 0, st>>>(flags, full_vocab);
    if (idtype == ANE_ID_U16) vocab_mark_kernel<uint16_t><<<flat_grid(n_tokens), 256, 0, st>>>(flags, tokens, n_tokens, full_vocab, ctx().status);
    else vocab_mark_kernel<int32_t><<<flat_grid(n_tokens), 256, 0, st>>>(flags, tokens, n_tokens, full_vocab, ctx().status);
    ANE_CUDA_TRY(cub::DeviceScan::ExclusiveSum(ws + 2 * ints, cub_bytes, flags, scan, full_vocab, st));
    vocab_assign_kernel<<<vb, 256, 0, st>>>(full_to_compact, compact_to_full, compact_vocab, flags, scan, full_vocab);
    ANE_LAUNCH_OK(3);
    return ANE_CUDA_OK;
}

static int vocab_rows(int mode, void *stream, float *full, float *compact, const int *compact_to_full, const int *count_dev,
                      int count_max, int dim, int full_vocab, const char *who) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(full && compact && compact_to_full, "%s: null pointer", who);
    ANE_REQUIRE(count_max >= 0 && dim >= 1 && full_vocab >= 1, "%s: bad sizes", who);
    if (count_max == 0) return ANE_CUDA_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = flat_grid((size_t)count_max * 32);
    if (mode == 0) vocab_rows_kernel<0><<<grid, LY_THREADS, 0, st>>>(full, compact, compact_to_full, count_dev, count_max, dim, full_vocab);
    else if (mode == 1) vocab_rows_kernel<1><<<grid, LY_THREADS, 0, st>>>(full, compact, compact_to_full, count_dev, count_max, dim, full_vocab);
    else vocab_rows_kernel<2><<<grid, LY_THREADS, 0, st>>>(full, compact, compact_to_full, count_dev, count_max, dim, full_vocab);
    ANE_LAUNCH_OK(1);
    return ANE_CUDA_OK;
}

int ane_cuda_vocab_compact_embed_dev(void *stream, float *compact_embed, const float *full_embed, const int *compact_to_full,
                                     const int *compact_vocab_dev, int compact_vocab_max, int dim, int full_vocab) {
    return vocab_rows(0, stream, const_cast<float *>(full_embed), compact_embed, compact_to_full, compact_vocab_dev, compact_vocab_max, dim,
                      full_vocab, __func__);
}
int ane_cuda_vocab_scatter_grads_dev(void *stream, float *full_gembed, const float *compact_gembed, const int *compact_to_full,
                                     const int *compact_vocab_dev, int compact_vocab_max, int dim, int full_vocab) {
    return vocab_rows(1, stream, full_gembed, const_cast<float *>(compact_gembed), compact_to_full, compact_vocab_dev, compact_vocab_max,
                      dim, full_vocab, __func__);
}
int ane_cuda_vocab_update_full_dev(void *stream, float *full_embed, const float *compact_embed, const int *compact_to_full,
                                   const int *compact_vocab_dev, int compact_vocab_max, int dim, int full_vocab) {
    return vocab_rows(2, stream, full_embed, const_cast<float *>(compact_embed), compact_to_full, compact_vocab_dev, compact_vocab_max, dim,
                      full_vocab, __func__);
}

}  // extern "C"
