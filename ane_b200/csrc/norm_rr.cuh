// norm_rr.cuh -- register-resident RMSNorm kernels.
//
// The two-sweep kernels of norm.cu read every tensor twice (the second time from L2) and keep
// only four 16-byte loads per tensor in flight per thread.  Here a block owns a [C x LG*VEC]
// token tile and every thread issues ALL of its loads for the tile before the first use --
// NV independent 16-byte loads per thread -- and keeps the raw
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
    dep_sync();

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

}  // namespace ane
