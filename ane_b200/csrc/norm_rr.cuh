// norm_rr.cuh -- register-resident RMSNorm kernels.
//
// The two-sweep kernels of norm.cu read every tensor twice (the second time from L2) and keep
// only four 16-byte loads per tensor in flight per thread.  Here a block owns a [C x LG*VEC]
// token tile and every thread issues ALL of its loads for the tile before the first use --
// NV (forward) or 2*NV (backward) independent 16-byte loads per thread -- and keeps the raw
// vectors in registers between the per-token reduction and the store.  HBM and L2 both see
// each byte once.  Channel c of the tile belongs to thread row group (c mod R), so one
// warp-level load instruction covers 32/LG adjacent channel rows.
#pragma once
#include "common.cuh"

namespace ane {

// out = (x * rrms) * w ; optional fused x2 = f*alpha + x (stored, then normalised).
template <typename T, int LG, int THREADS, int NV, bool FUSE_RES>
__global__ void __launch_bounds__(THREADS)
rmsnorm_fwd_rr_kernel(T *out, T *x2out, const T *x, const T *f, const float *__restrict__ w, int C, int S,
                      int tiles_per_seq, float alpha, float eps) {
    constexpr int VEC = Elt<T>::VEC;
    constexpr int R = THREADS / LG;
    constexpr int TW = LG * VEC;
    __shared__ __align__(16) float red[R][TW];
    __shared__ __align__(16) float tot[TW];

    const int b = blockIdx.x / tiles_per_seq;
    const int lg = threadIdx.x % LG, rg = threadIdx.x / LG;
    const int t = (blockIdx.x % tiles_per_seq) * TW + lg * VEC;
    const bool active = t < S;
    const size_t base = (size_t)b * C * S + t + (size_t)rg * S;
    const size_t step = (size_t)R * S;

    Raw<T, VEC> r[NV];
    V<VEC> ss = V<VEC>::splat(0.0f);

    if (!FUSE_RES) {
#pragma unroll
        for (int k = 0; k < NV; k++)
            if (active && k * R + rg < C) r[k].load_stream(x + base + k * step);
#pragma unroll
        for (int k = 0; k < NV; k++)
            if (active && k * R + rg < C) { const V<VEC> v = r[k].get(); ss = vfma(v, v, ss); }
    } else {
        constexpr int UB = NV < 8 ? NV : 8;          // x and f in batches of UB channels
        #pragma unroll
        for (int k0 = 0; k0 < NV; k0 += UB) {
            Raw<T, VEC> rf[UB];
#pragma unroll
            for (int u = 0; u < UB; u++) {
                const int k = k0 + u;
                if (k < NV && active && k * R + rg < C) {
                    r[k].load_stream(x + base + k * step);
                    rf[u].load_stream(f + base + k * step);
                }
            }
#pragma unroll
            for (int u = 0; u < UB; u++) {
                const int k = k0 + u;
                if (k < NV && active && k * R + rg < C) {
                    r[k].put(vadd(vscale(rf[u].get(), alpha), r[k].get()));      // train.m:460, two roundings
                    r[k].store_stream(x2out + base + k * step);
                    const V<VEC> v = r[k].get();                                  // the stored (rounded) value
                    ss = vfma(v, v, ss);
                }
            }
        }
    }
    lanes_to_smem<VEC>(&red[rg][lg * VEC], ss);
    __syncthreads();
    {   // column sums with the whole block, then rrms once per token
        constexpr int P = THREADS / TW;
        const float s = block_column_sum<R, TW, THREADS>(&red[0][0], threadIdx.x);
        if (threadIdx.x % P == 0) tot[threadIdx.x / P] = 1.0f / sqrtf(__fadd_rn(__fmul_rn(s, 1.0f / (float)C), eps));
    }
    __syncthreads();
    if (!active) return;
    const V<VEC> rr = lanes_from_smem<VEC>(&tot[lg * VEC]);
#pragma unroll
    for (int k = 0; k < NV; k++) {
        const int c = k * R + rg;
        if (c < C) {
            Raw<T, VEC> o;
            o.put(vscale(vmul(r[k].get(), rr), __ldg(w + c)));      // stories_cpu_ops.h:16-19
            o.store_stream(out + base + k * step);
        }
    }
}

// dx = rmsnorm_bwd(dy, x, w) [+ add]; dw partials per persistent block (see norm.cu).
template <typename T, int LG, int THREADS, int NV, bool HAS_ADD>
__global__ void __launch_bounds__(THREADS)
rmsnorm_bwd_rr_kernel(T *dx, float *__restrict__ partial, const T *dy, const T *x, const float *__restrict__ w,
                      const T *add, int C, int S, int tiles_per_seq, int ntiles, float eps, unsigned flags) {
    constexpr int VEC = Elt<T>::VEC;
    constexpr int R = THREADS / LG;
    constexpr int TW = LG * VEC;
    __shared__ __align__(16) float red[2][R][TW];
    __shared__ __align__(16) float tot[2][TW];
    extern __shared__ float dwacc[];  // [C]

    const int lg = threadIdx.x % LG, rg = threadIdx.x / LG;
    const float invd = 1.0f / (float)C;
    const bool exact = (flags & ANE_NORM_BWD_EXACT) != 0;
    const size_t step = (size_t)R * S;

    for (int c = threadIdx.x; c < C; c += THREADS) dwacc[c] = 0.0f;
    __syncthreads();

    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int b = tile / tiles_per_seq;
        const int t = (tile % tiles_per_seq) * TW + lg * VEC;
        const bool active = t < S;
        const size_t base = (size_t)b * C * S + t + (size_t)rg * S;

        Raw<T, VEC> rx[NV], rd[NV];
#pragma unroll
        for (int k = 0; k < NV; k++) {
            if (active && k * R + rg < C) {
                rx[k].load_stream(x + base + k * step);
                rd[k].load_stream(dy + base + k * step);
            }
        }
        V<VEC> ss = V<VEC>::splat(0.0f), dot = V<VEC>::splat(0.0f);
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const int c = k * R + rg;
            if (active && c < C) {
                const V<VEC> xv = rx[k].get(), dv = rd[k].get();
                ss = vfma(xv, xv, ss);
                dot = vfma_s(vmul(dv, xv), __ldg(w + c), dot);      // stories_cpu_ops.h:35-38
            }
        }
        lanes_to_smem<VEC>(&red[0][rg][lg * VEC], ss);
        lanes_to_smem<VEC>(&red[1][rg][lg * VEC], dot);
        __syncthreads();
        {   // column sums with the whole block, then rrms and coef once per token
            constexpr int P = THREADS / TW;
            const float s0 = block_column_sum<R, TW, THREADS>(&red[0][0][0], threadIdx.x);
            const float s1 = block_column_sum<R, TW, THREADS>(&red[1][0][0], threadIdx.x);
            if (threadIdx.x % P == 0) {
                const float r1 = 1.0f / sqrtf(__fadd_rn(__fmul_rn(s0, invd), eps));
                float r2 = r1 * r1;
                r2 = r2 * invd;
                tot[0][threadIdx.x / P] = r1;
                tot[1][threadIdx.x / P] = s1 * r2;                                 // stories_cpu_ops.h:39-41
            }
        }
        __syncthreads();
        const V<VEC> rr = lanes_from_smem<VEC>(&tot[0][lg * VEC]), coef = lanes_from_smem<VEC>(&tot[1][lg * VEC]);
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const int c = k * R + rg;
            float dwp = 0.0f;
            if (active && c < C) {
                Raw<T, VEC> ra;
                if (HAS_ADD) ra.load_stream(add + base + k * step);
                const V<VEC> xv = rx[k].get(), dv = rd[k].get();
                const float wc = __ldg(w + c);
                V<VEC> o;
                if (exact) o = vmul(vsub(vscale(dv, wc), vmul(xv, coef)), rr);
                else o = vscale(vmul(vsub(dv, vmul(xv, coef)), rr), wc);             // stories_cpu_ops.h:43-46
                dwp = vmul(vmul(dv, xv), rr).hsum();                                // stories_cpu_ops.h:47-50
                if (HAS_ADD) o = vadd(o, ra.get());                                 // train.m:590,721
                Raw<T, VEC> ro;
                ro.put(o);
                ro.store_stream(dx + base + k * step);
            }
#pragma unroll
            for (int off = LG / 2; off > 0; off >>= 1) dwp += __shfl_xor_sync(0xffffffffu, dwp, off);
            if (lg == 0 && c < C) dwacc[c] += dwp;       // row group rg is the only writer of channel c
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += THREADS) partial[(size_t)blockIdx.x * C + c] = dwacc[c];
}

}  // namespace ane
