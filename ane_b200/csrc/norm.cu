// norm.cu -- RMSNorm forward / backward over channel-first [B][C][S] tensors, with the
// DeepNet residual fused in front of the forward and the residual-gradient add fused behind
// the backward.
//
// Data layout and work split.  S is the contiguous axis, the reduction runs over C with
// stride S.  A block owns a token tile of LG*VEC tokens of one sequence: LG adjacent lanes
// cover the tile with 16-byte loads and THREADS/LG "row groups" stride over the channels.
// Per-token partial sums meet in shared memory.  Two families:
//   * two-sweep kernels (this file): each tensor is swept twice (reduce, then normalise); a
//     block's tile is at most a few hundred KB, so the second sweep is served by L2 and HBM
//     sees every input byte once.  Any C, any alignment (VEC = 1 path).
//   * register-resident kernels (norm_rr.cuh): the whole tile stays in registers between
//     the reduction and the store; used when C fits the per-thread budget.
// The per-element math runs on packed fp32 pairs (V<VEC>, common.cuh).
//
// dw (a sum over all tokens) is made deterministic without float atomics: the backward kernel
// is persistent, every block keeps dw partials for its tiles in shared memory in a fixed tile
// order, writes them to a scratch matrix [blocks][C], and a second kernel adds the rows in
// block order.
#include "common.cuh"
#include "norm_rr.cuh"
#include "norm_st.cuh"

namespace ane {

constexpr int NORM_THREADS = 256;
constexpr int NORM_U = 4;  // channel rows in flight per thread and tensor

template <typename T, int VEC, int LG, bool FUSE_RES>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(T *out, T *x2out, const T *x, const T *f,
                   const float *__restrict__ w, int C, int S, int tiles_per_seq, float alpha, float eps) {
    constexpr int R = NORM_THREADS / LG;
    constexpr int TW = LG * VEC;
    __shared__ __align__(16) float red[R][TW];
    __shared__ __align__(16) float tot[TW];

    const int b = blockIdx.x / tiles_per_seq;
    const int t0 = (blockIdx.x % tiles_per_seq) * TW;
    const int lg = threadIdx.x % LG, rg = threadIdx.x / LG;
    const int t = t0 + lg * VEC;
    const bool active = t < S;
    const size_t base = (size_t)b * C * S + t + (size_t)rg * S;
    const size_t step = (size_t)R * S;
    
    V<VEC> ss = V<VEC>::splat(0.0f);

    // sweep 1: sum of squares (and, when fused, x2 = f*alpha + x written out)
    for (int cb = 0; cb < C; cb += R * NORM_U) {
        Raw<T, VEC> rx[NORM_U], rf[NORM_U];
#pragma unroll
        for (int u = 0; u < NORM_U; u++) {
            const int c = cb + u * R + rg;
            if (active && c < C) {
                const size_t o = base + (size_t)(cb / R + u) * step;
                if (FUSE_RES) {
                    rx[u].load_stream(x + o);
                    rf[u].load_stream(f + o);
                } else {
                    rx[u].load(x + o);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < NORM_U; u++) {
            const int c = cb + u * R + rg;
            if (active && c < C) {
                V<VEC> v = rx[u].get();
                if (FUSE_RES) {
                    v = vadd(vscale(rf[u].get(), alpha), v);              // train.m:460, two roundings
                    Raw<T, VEC> o;
                    o.put(v);
                    o.store(x2out + base + (size_t)(cb / R + u) * step);   // stays in L2 for sweep 2
                    v = o.get();                                          // the stored (rounded) value
                }
                ss = vfma(v, v, ss);
            }
        }
    }
    lanes_to_smem<VEC>(&red[rg][lg * VEC], ss);
    __syncthreads();
    {   // column sums with the whole block, then rrms once per token
        constexpr int P = NORM_THREADS / TW;
        const float s = block_column_sum<R, TW, NORM_THREADS>(&red[0][0], threadIdx.x);
        if (threadIdx.x % P == 0) tot[threadIdx.x / P] = 1.0f / sqrtf(__fadd_rn(__fmul_rn(s, 1.0f / (float)C), eps));
    }
    __syncthreads();
    const V<VEC> rr = lanes_from_smem<VEC>(&tot[lg * VEC]);

    // sweep 2: out = (x * rrms) * w[c]          (stories_cpu_ops.h:16-19, in that order)
    const T *src = FUSE_RES ? x2out : x;
    for (int cb = 0; cb < C; cb += R * NORM_U) {
        Raw<T, VEC> rx[NORM_U];
#pragma unroll
        for (int u = 0; u < NORM_U; u++) {
            const int c = cb + u * R + rg;
            if (active && c < C) {
                const size_t o = base + (size_t)(cb / R + u) * step;
                if (FUSE_RES) rx[u].load(src + o);
                else rx[u].load_stream(src + o);
            }
        }
#pragma unroll
        for (int u = 0; u < NORM_U; u++) {
            const int c = cb + u * R + rg;
            if (active && c < C) {
                const V<VEC> v = vscale(vmul(rx[u].get(), rr), __ldg(w + c));
                Raw<T, VEC> o;
                o.put(v);
                o.store_stream(out + base + (size_t)(cb / R + u) * step);
            }
        }
    }
}

template <typename T, int VEC, int LG, bool HAS_ADD>
__global__ void __launch_bounds__(NORM_THREADS, 2)
rmsnorm_bwd_kernel(T *dx, float *__restrict__ partial, const T *dy, const T *x,
                   const float *__restrict__ w, const T *add, int C, int S, int tiles_per_seq,
                   int ntiles, float eps, unsigned flags) {
    constexpr int R = NORM_THREADS / LG;
    constexpr int TW = LG * VEC;
    __shared__ __align__(16) float red[2][R][TW];
    __shared__ __align__(16) float tot[2][TW];
    extern __shared__ float dwacc[];  // [C]

    const int lg = threadIdx.x % LG, rg = threadIdx.x / LG;
    const float invd = 1.0f / (float)C;
    const bool exact = (flags & ANE_NORM_BWD_EXACT) != 0;
    const size_t step = (size_t)R * S;

    for (int c = threadIdx.x; c < C; c += NORM_THREADS) dwacc[c] = 0.0f;
    __syncthreads();

    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int b = tile / tiles_per_seq;
        const int t = (tile % tiles_per_seq) * TW + lg * VEC;
        const bool active = t < S;
        const size_t base = (size_t)b * C * S + t + (size_t)rg * S;

        V<VEC> ss = V<VEC>::splat(0.0f), dot = V<VEC>::splat(0.0f);

        // sweep 1: ss = sum x^2 ; dot = sum (dy*x)*w       (stories_cpu_ops.h:26-38)
        for (int cb = 0; cb < C; cb += R * NORM_U) {
            Raw<T, VEC> rx[NORM_U], rd[NORM_U];
#pragma unroll
            for (int u = 0; u < NORM_U; u++) {
                const int c = cb + u * R + rg;
                if (active && c < C) {
                    const size_t o = base + (size_t)(cb / R + u) * step;
                    rx[u].load(x + o);
                    rd[u].load(dy + o);
                }
            }
#pragma unroll
            for (int u = 0; u < NORM_U; u++) {
                const int c = cb + u * R + rg;
                if (active && c < C) {
                    const V<VEC> xv = rx[u].get(), dv = rd[u].get();
                    ss = vfma(xv, xv, ss);
                    dot = vfma_s(vmul(dv, xv), __ldg(w + c), dot);
                }
            }
        }
        lanes_to_smem<VEC>(&red[0][rg][lg * VEC], ss);
        lanes_to_smem<VEC>(&red[1][rg][lg * VEC], dot);
        __syncthreads();
        {   // column sums with the whole block, then rrms and coef once per token
            constexpr int P = NORM_THREADS / TW;
            const float s0 = block_column_sum<R, TW, NORM_THREADS>(&red[0][0][0], threadIdx.x);
            const float s1 = block_column_sum<R, TW, NORM_THREADS>(&red[1][0][0], threadIdx.x);
            if (threadIdx.x % P == 0) {
                const float r1 = 1.0f / sqrtf(__fadd_rn(__fmul_rn(s0, invd), eps));
                float r2 = r1 * r1;
                r2 = r2 * invd;
                tot[0][threadIdx.x / P] = r1;
                tot[1][threadIdx.x / P] = s1 * r2;            // stories_cpu_ops.h:39-41
            }
        }
        __syncthreads();
        const V<VEC> rr = lanes_from_smem<VEC>(&tot[0][lg * VEC]), coef = lanes_from_smem<VEC>(&tot[1][lg * VEC]);

        // sweep 2: dx and the dw partials (inputs come back from L2)
        for (int cb = 0; cb < C; cb += R * NORM_U) {
            Raw<T, VEC> rx[NORM_U], rd[NORM_U], ra[NORM_U];
#pragma unroll
            for (int u = 0; u < NORM_U; u++) {
                const int c = cb + u * R + rg;
                if (active && c < C) {
                    const size_t o = base + (size_t)(cb / R + u) * step;
                    rx[u].load_stream(x + o);
                    rd[u].load_stream(dy + o);
                    if (HAS_ADD) ra[u].load_stream(add + o);
                }
            }
#pragma unroll
            for (int u = 0; u < NORM_U; u++) {
                const int c = cb + u * R + rg;
                float dwp = 0.0f;
                if (active && c < C) {
                    const V<VEC> xv = rx[u].get(), dv = rd[u].get();
                    const float wc = __ldg(w + c);
                    V<VEC> o;
                    if (exact) o = vmul(vsub(vscale(dv, wc), vmul(xv, coef)), rr);
                    else o = vscale(vmul(vsub(dv, vmul(xv, coef)), rr), wc);     // stories_cpu_ops.h:43-46
                    dwp = vmul(vmul(dv, xv), rr).hsum();                        // stories_cpu_ops.h:47-50
                    if (HAS_ADD) o = vadd(o, ra[u].get());                      // train.m:590,721
                    Raw<T, VEC> ro;
                    ro.put(o);
                    ro.store_stream(dx + base + (size_t)(cb / R + u) * step);
                }
                // sum over the LG lanes that share channel c (the loop is uniform across the warp)
#pragma unroll
                for (int off = LG / 2; off > 0; off >>= 1) dwp += __shfl_xor_sync(0xffffffffu, dwp, off);
                if (lg == 0 && c < C) dwacc[c] += dwp;   // row group rg is the only writer of channel c
            }
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += NORM_THREADS) partial[(size_t)blockIdx.x * C + c] = dwacc[c];
}

template <typename T, bool FUSE_RES>
static int launch_rmsnorm_fwd(cudaStream_t st, int B, int C, int S, void *out, void *x2, const void *x, const void *f,
                              const float *w, float alpha, float eps) {
    constexpr int VEC = Elt<T>::VEC;
    const bool vec = (S % VEC == 0) && aligned16(out) && aligned16(x) && (!FUSE_RES || (aligned16(x2) && aligned16(f)));
    if (vec) {
        // register-resident path: tile shape by knob, NV = channels per thread (compile-time bound)
#define ANE_FWD_RR(LGv, THv, NVv)                                                                                   \
        do {                                                                                                        \
            const int tps_ = (S + (LGv) * VEC - 1) / ((LGv) * VEC);                                                  \
            launch_dep(DEP_NORM_FWD, rmsnorm_fwd_rr_kernel<T, LGv, THv, NVv, FUSE_RES>, dim3((unsigned)(B * tps_)), dim3(THv), 0, st, \
                       (T *)out, (T *)x2, (const T *)x, (const T *)f, w, C, S, tps_, alpha, eps);                   \
            ANE_LAUNCH_OK(1);                                                                                       \
            return ANE_CUDA_OK;                                                                                     \
        } while (0)
#define ANE_FWD_RR_NV(LGv, THv)                                                                                     \
        do {                                                                                                        \
            const int nv_ = (C + (THv) / (LGv) - 1) / ((THv) / (LGv));                                               \
            if (nv_ <= 4) ANE_FWD_RR(LGv, THv, 4);                                                                  \
            else if (nv_ <= 8) ANE_FWD_RR(LGv, THv, 8);                                                             \
            else if (nv_ <= 12) ANE_FWD_RR(LGv, THv, 12);                                                           \
            else if (nv_ <= 16) ANE_FWD_RR(LGv, THv, 16);                                                           \
        } while (0)
        // Measured on B200 (C = 1024, bf16): the shared-memory strip wins for the plain forward (71-89 % of the
        // copy rate), the 512-thread register-resident tile for the fused residual form (76-93 %).
        const int knob_f = tuning("norm_fwd", FUSE_RES ? 4 : 6);
        if (knob_f == 6 && (size_t)C * 64 <= 160 * 1024) {        // shared-memory-resident strip, 64-byte rows
            constexpr int LGs = 4;
            const int tps_ = (S + LGs * VEC - 1) / (LGs * VEC);
            const size_t smem = (size_t)C * LGs * 16;
            auto k_ = rmsnorm_fwd_st_kernel<T, LGs, FUSE_RES>;
            ANE_CUDA_TRY(cudaFuncSetAttribute(k_, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            launch_dep(DEP_NORM_FWD, k_, dim3((unsigned)(B * tps_)), dim3(ST_THREADS), smem, st, (T *)out, (T *)x2, (const T *)x, (const T *)f, w, C, S, tps_, alpha, eps);
            ANE_LAUNCH_OK(1);
            return ANE_CUDA_OK;
        }
        switch (knob_f) {
            case 2: ANE_FWD_RR_NV(4, 256); break;        // C <= 1024
            case 3: ANE_FWD_RR_NV(4, 512); break;        // C <= 2048
            case 4: ANE_FWD_RR_NV(8, 512); break;        // C <= 1024, 128-byte row segments
            default: break;
        }
#undef ANE_FWD_RR_NV
#undef ANE_FWD_RR
        constexpr int LG = 8;
        const int tps = (S + LG * VEC - 1) / (LG * VEC);
        rmsnorm_fwd_kernel<T, VEC, LG, FUSE_RES><<<(unsigned)(B * tps), NORM_THREADS, 0, st>>>(
            (T *)out, (T *)x2, (const T *)x, (const T *)f, w, C, S, tps, alpha, eps);
    } else {
        constexpr int LG = 32;
        const int tps = (S + LG - 1) / LG;
        rmsnorm_fwd_kernel<T, 1, LG, FUSE_RES><<<(unsigned)(B * tps), NORM_THREADS, 0, st>>>(
            (T *)out, (T *)x2, (const T *)x, (const T *)f, w, C, S, tps, alpha, eps);
    }
    ANE_LAUNCH_OK(1);
    return ANE_CUDA_OK;
}

template <typename KernelT>
static int persistent_grid(KernelT kernel, int threads, size_t dyn_smem, int ntiles) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, dyn_smem) != cudaSuccess || per_sm < 1)
        per_sm = 1;
    long g = (long)per_sm * ctx().sm_count;
    if (g > ntiles) g = ntiles;
    if (g < 1) g = 1;
    return (int)g;
}

// The cluster forms of the backward: CL blocks share the channels of one token tile (norm_st.cuh).
template <typename T, bool HAS_ADD, int LGs, int CL, int NBUF>
static int launch_rmsnorm_bwd_cluster(cudaStream_t st, int B, int C, int S, void *dx, float *dw, const void *dy, const void *x,
                                      const float *w, const void *add, float eps, unsigned flags) {
    constexpr int VEC = Elt<T>::VEC;
    const int tps_ = (S + LGs * VEC - 1) / (LGs * VEC);
    const int ntiles = B * tps_;
    const int part = (C + CL - 1) / CL;
    const size_t smem_st = (size_t)2 * NBUF * part * LGs * 16 + (size_t)part * sizeof(float);
    auto k_ = rmsnorm_bwd_cluster_kernel<T, LGs, HAS_ADD, CL, NBUF>;
    ANE_CUDA_TRY(cudaFuncSetAttribute(k_, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_st));
    static int max_clusters = 0;               // co-resident clusters of this instantiation at the last smem size
    static size_t max_clusters_smem = 0;
    if (max_clusters == 0 || max_clusters_smem != smem_st) {
        cudaLaunchConfig_t q = {};
        q.gridDim = dim3(CL * ctx().sm_count * 4, 1, 1);
        q.blockDim = dim3(ST_THREADS, 1, 1);
        q.dynamicSmemBytes = smem_st;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, k_, &q) != cudaSuccess || n < 1) { cudaGetLastError(); n = ctx().sm_count / CL; }
        max_clusters = n;
        max_clusters_smem = smem_st;
    }
    const int ngroups = max_clusters < ntiles ? max_clusters : ntiles;
    float *partial = static_cast<float *>(workspace((size_t)ngroups * C * sizeof(float)));
    if (!partial) return fail(ANE_CUDA_ERR_NOMEM, "rmsnorm_bwd: no scratch for %d x %d partials", ngroups, C);
    launch_dep(DEP_NORM_BWD, k_, dim3((unsigned)(CL * ngroups)), dim3(ST_THREADS), smem_st, st, (T *)dx, partial, (const T *)dy, (const T *)x, w, (const T *)add, C, S, tps_, ntiles, eps, flags);
    launch_dep(DEP_COLSUM, column_sum_add_kernel<>, dim3((C + 31) / 32), dim3(256), 0, st, dw, (const float *)partial, ngroups, C);
    ANE_LAUNCH_OK(2);
    return ANE_CUDA_OK;
}

template <typename T, bool HAS_ADD>
static int launch_rmsnorm_bwd(cudaStream_t st, int B, int C, int S, void *dx, float *dw, const void *dy, const void *x,
                              const float *w, const void *add, float eps, unsigned flags) {
    constexpr int VEC = Elt<T>::VEC;
    const bool vec = (S % VEC == 0) && aligned16(dx) && aligned16(dy) && aligned16(x) && (!HAS_ADD || aligned16(add));
    const size_t smem = (size_t)C * sizeof(float);
    int grid, ntiles;
    float *partial;
    if (vec) {
        // Measured on B200, fraction of the copy rate (bf16 C = 1024 at 32 / 64 sequences; fp32 C = 768 x 256 at 1024 sequences):
        //   pair of blocks, 64-byte rows (8)              0.65 / 0.72, with add 0.60 / 0.64; fp32 0.53, with add 0.62
        //   cluster of four, 128-byte rows (10)           0.64 / 0.70, with add 0.68 / 0.73; fp32 0.65, with add 0.72
        //   cluster of four, 64-byte rows, two strips (9) 0.55 / 0.58, with add 0.53 / 0.54; fp32 0.63, with add 0.64
        //   cluster of eight, 256-byte rows (11)          0.50 / 0.54, with add 0.59 / 0.62; fp32 0.68, with add 0.77
        //   two-sweep kernel below (0)                    0.41 - 0.58
        // The width of a row segment decides: the same kernel with more warps, fewer instructions, the next tile always in
        // flight or the rows to add prefetched runs at the same speed, wider rows run faster until the cluster gets too
        // large to place.  (Also tried and removed: a register-resident tile, 0.37-0.50; one block per strip with 32- or
        // 64-byte rows, 0.37-0.53; a statistics kernel followed by an element-wise kernel, 0.42-0.57.)
        // fp32 over many tiles gains another 3-6 % from 256-byte rows (C = 768 and 1024, 256 sequences and more)
        const bool wide_f32 = sizeof(T) == 4 && C >= 512 && (long long)B * ((S + 63) / 64) >= 256;
        const int knob_b = tuning("norm_bwd", wide_f32 ? 11 : (HAS_ADD || sizeof(T) == 4) ? 10 : 8);
        if (knob_b == 11 && C >= 512 && (size_t)C * 66 <= 200 * 1024)           // channel eighths on a cluster of eight, 256-byte rows
            return launch_rmsnorm_bwd_cluster<T, HAS_ADD, 16, 8, 1>(st, B, C, S, dx, dw, dy, x, w, add, eps, flags);
        if (knob_b == 12 && C >= 512 && (size_t)C * 66 <= 200 * 1024)           // channel eighths, 128-byte rows, two strip pairs: the next tile always in flight
            return launch_rmsnorm_bwd_cluster<T, HAS_ADD, 8, 8, 2>(st, B, C, S, dx, dw, dy, x, w, add, eps, flags);
        if ((knob_b == 9 || knob_b == 10) && C >= 256 && (size_t)C * 66 <= 200 * 1024) {
            // channel quarters on a cluster of four: 64-byte rows with double-buffered strips (9), or 128-byte rows (10)
            if (knob_b == 9) return launch_rmsnorm_bwd_cluster<T, HAS_ADD, 4, 4, 2>(st, B, C, S, dx, dw, dy, x, w, add, eps, flags);
            return launch_rmsnorm_bwd_cluster<T, HAS_ADD, 8, 4, 1>(st, B, C, S, dx, dw, dy, x, w, add, eps, flags);
        }
        if ((knob_b >= 8) && (size_t)C * 66 <= 200 * 1024 && C >= 64) {      // channel halves on a pair of blocks, 64-byte rows
            constexpr int LGs = 4;
            const int tps_ = (S + LGs * VEC - 1) / (LGs * VEC);
            ntiles = B * tps_;
            const int half = (C + 1) / 2;
            const size_t smem_st = (size_t)2 * half * LGs * 16 + (size_t)half * sizeof(float);
            auto k_ = rmsnorm_bwd_pair_kernel<T, LGs, HAS_ADD>;
            ANE_CUDA_TRY(cudaFuncSetAttribute(k_, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_st));
            int per_sm = (int)((220 * 1024) / (smem_st + 5 * 1024));
            per_sm = per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm);
            int npairs = per_sm * ctx().sm_count / 2;
            if (npairs > ntiles) npairs = ntiles;
            partial = static_cast<float *>(workspace((size_t)npairs * C * sizeof(float)));
            if (!partial) return fail(ANE_CUDA_ERR_NOMEM, "rmsnorm_bwd: no scratch for %d x %d partials", npairs, C);
            launch_dep(DEP_NORM_BWD, k_, dim3((unsigned)(2 * npairs)), dim3(ST_THREADS), smem_st, st, (T *)dx, partial, (const T *)dy, (const T *)x, w, (const T *)add, C, S, tps_, ntiles, eps, flags);
            launch_dep(DEP_COLSUM, column_sum_add_kernel<>, dim3((C + 31) / 32), dim3(256), 0, st, dw, (const float *)partial, npairs, C);
            ANE_LAUNCH_OK(2);
            return ANE_CUDA_OK;
        }
        constexpr int LG = 8;
        auto k = rmsnorm_bwd_kernel<T, VEC, LG, HAS_ADD>;
        const int tps = (S + LG * VEC - 1) / (LG * VEC);
        ntiles = B * tps;
        grid = persistent_grid(k, NORM_THREADS, smem, ntiles);
        partial = static_cast<float *>(workspace((size_t)grid * C * sizeof(float)));
        if (!partial) return fail(ANE_CUDA_ERR_NOMEM, "rmsnorm_bwd: no scratch for %d x %d partials", grid, C);
        k<<<grid, NORM_THREADS, smem, st>>>((T *)dx, partial, (const T *)dy, (const T *)x, w, (const T *)add, C, S, tps,
                                            ntiles, eps, flags);
    } else {
        constexpr int LG = 32;
        auto k = rmsnorm_bwd_kernel<T, 1, LG, HAS_ADD>;
        const int tps = (S + LG - 1) / LG;
        ntiles = B * tps;
        grid = persistent_grid(k, NORM_THREADS, smem, ntiles);
        partial = static_cast<float *>(workspace((size_t)grid * C * sizeof(float)));
        if (!partial) return fail(ANE_CUDA_ERR_NOMEM, "rmsnorm_bwd: no scratch for %d x %d partials", grid, C);
        k<<<grid, NORM_THREADS, smem, st>>>((T *)dx, partial, (const T *)dy, (const T *)x, w, (const T *)add, C, S, tps,
                                            ntiles, eps, flags);
    }
    column_sum_add_kernel<><<<(C + 31) / 32, 256, 0, st>>>(dw, partial, grid, C);
    ANE_LAUNCH_OK(2);
    return ANE_CUDA_OK;
}

// Shared by the per-head operators, which treat [B][heads*hd][S] as [B*heads][hd][S].
int rmsnorm_fwd_any(cudaStream_t st, ane_dtype dtype, int B, int C, int S, void *out, const void *x, const float *w, float eps) {
    ANE_DISPATCH_DTYPE(dtype, T, return (launch_rmsnorm_fwd<T, false>(st, B, C, S, out, nullptr, x, nullptr, w, 0.0f, eps)));
    return ANE_CUDA_OK;
}
int rmsnorm_bwd_any(cudaStream_t st, ane_dtype dtype, int B, int C, int S, void *dx, float *dw, const void *dy,
                    const void *x, const float *w, const void *add, float eps, unsigned flags) {
    if (add) {
        ANE_DISPATCH_DTYPE(dtype, T, return (launch_rmsnorm_bwd<T, true>(st, B, C, S, dx, dw, dy, x, w, add, eps, flags)));
    } else {
        ANE_DISPATCH_DTYPE(dtype, T, return (launch_rmsnorm_bwd<T, false>(st, B, C, S, dx, dw, dy, x, w, nullptr, eps, flags)));
    }
    return ANE_CUDA_OK;
}

static int check_bcs(const char *fn, int B, int C, int S) {
    if (B < 1 || C < 1 || S < 1) return fail(ANE_CUDA_ERR_INVALID, "%s: B, C, S must be positive (got %d, %d, %d)", fn, B, C, S);
    if (C > 8192) return fail(ANE_CUDA_ERR_UNSUPPORTED, "%s: C = %d exceeds 8192", fn, C);
    if ((long long)B * ((S + 7) / 8) > 0x7fffffffLL) return fail(ANE_CUDA_ERR_UNSUPPORTED, "%s: too many token tiles", fn);
    return ANE_CUDA_OK;
}


// ------------------------------------------------------------------ allocation-free backward
// The backward kernel needs a [blocks][C] matrix of dw partials.  The regular entry point takes
// it from the library's grow-only scratch range, i.e. it may call cudaMalloc.  Some callers
// cannot tolerate that: a host process whose framework has already reserved the whole device
// for its own caching pool (a cudaMalloc from a side library then fails or fragments the
// pool), or a latency-critical loop that must never hit cudaMalloc's device-wide
// synchronisation.  For them the same kernels run with the partials in a fixed array that is
// part of the module image: every GPU that loads this library holds
// STATIC_MAX_BLOCKS * STATIC_MAX_C * 4 bytes (2.3 MiB) of it from load until the process exits.
constexpr int STATIC_MAX_C = 2048;
constexpr int STATIC_MAX_BLOCKS = 296;   // two resident blocks per SM on a 148-SM part
static __device__ __align__(256) float g_static_dw_partials[(size_t)STATIC_MAX_BLOCKS * STATIC_MAX_C];

// In host code the array's name is only a handle for the runtime, not a device address; the
// address has to be asked for, per device, with that device current.
constexpr int STATIC_MAX_DEVICES = 64;
static float *g_static_dw_addr[STATIC_MAX_DEVICES] = {};
static int g_static_sm_count[STATIC_MAX_DEVICES] = {};

static int static_scratch_for_current_device(float **addr, int *sm_count) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(ANE_CUDA_ERR_CUDA, "rmsnorm_bwd_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= STATIC_MAX_DEVICES) return fail(ANE_CUDA_ERR_UNSUPPORTED, "rmsnorm_bwd_static: device ordinal %d not supported", dev);
    if (!g_static_dw_addr[dev]) {       // first call on this device: resolve and remember
        int major = 0, sms = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return fail(ANE_CUDA_ERR_CUDA, "rmsnorm_bwd_static: cudaDeviceGetAttribute failed: %s", cudaGetErrorString(e));
        if (major != 10) return fail(ANE_CUDA_ERR_UNSUPPORTED, "rmsnorm_bwd_static: device %d is not sm_100 (the kernels are built for sm_100a only)", dev);
        float *p = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_static_dw_partials);
        if (e != cudaSuccess || !p) return fail(ANE_CUDA_ERR_CUDA, "rmsnorm_bwd_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_static_sm_count[dev] = sms;
        g_static_dw_addr[dev] = p;
    }
    *addr = g_static_dw_addr[dev];
    *sm_count = g_static_sm_count[dev];
    return ANE_CUDA_OK;
}

template <typename T, bool HAS_ADD>
static int launch_rmsnorm_bwd_static(cudaStream_t st, float *partial, int sm_count, int B, int C, int S, void *dx, float *dw,
                                     const void *dy, const void *x, const float *w, const void *add, float eps, unsigned flags) {
    constexpr int VEC = Elt<T>::VEC;
    const bool vec = (S % VEC == 0) && aligned16(dx) && aligned16(dy) && aligned16(x) && (!HAS_ADD || aligned16(add));
    const size_t smem = (size_t)C * sizeof(float);
    int cap = 2 * sm_count;
    if (cap > STATIC_MAX_BLOCKS) cap = STATIC_MAX_BLOCKS;
    int grid;
    if (vec) {
        constexpr int LG = 8;
        const int tps = (S + LG * VEC - 1) / (LG * VEC);
        const int ntiles = B * tps;
        grid = ntiles < cap ? ntiles : cap;
        rmsnorm_bwd_kernel<T, VEC, LG, HAS_ADD><<<grid, NORM_THREADS, smem, st>>>((T *)dx, partial, (const T *)dy, (const T *)x, w,
                                                                                 (const T *)add, C, S, tps, ntiles, eps, flags);
    } else {
        constexpr int LG = 32;
        const int tps = (S + LG - 1) / LG;
        const int ntiles = B * tps;
        grid = ntiles < cap ? ntiles : cap;
        rmsnorm_bwd_kernel<T, 1, LG, HAS_ADD><<<grid, NORM_THREADS, smem, st>>>((T *)dx, partial, (const T *)dy, (const T *)x, w,
                                                                               (const T *)add, C, S, tps, ntiles, eps, flags);
    }
    column_sum_add_kernel<><<<(C + 31) / 32, 256, 0, st>>>(dw, partial, grid, C);
    ANE_LAUNCH_OK(2);
    return ANE_CUDA_OK;
}

}  // namespace ane

using namespace ane;

extern "C" {

int ane_cuda_rmsnorm_dev(void *stream, ane_dtype dtype, int B, int C, int S, void *out, const void *x, const float *w,
                         float eps) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && x && w, "%s: null pointer", __func__);
    ANE_REQUIRE(dtype_ok(dtype), "%s: bad dtype", __func__);
    if (int rc = check_bcs(__func__, B, C, S)) return rc;
    ANE_CHECK_EXTENT(out, (size_t)B * C * S * dtype_size(dtype)); ANE_CHECK_EXTENT(x, (size_t)B * C * S * dtype_size(dtype)); ANE_CHECK_EXTENT(w, (size_t)C * 4);
    return rmsnorm_fwd_any((cudaStream_t)stream, dtype, B, C, S, out, x, w, eps);
}

int ane_cuda_residual_rmsnorm_dev(void *stream, ane_dtype dtype, int B, int C, int S, void *x2, void *x2norm,
                                  const void *x, const void *f, const float *w, float alpha, float eps) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(x2 && x2norm && x && f && w, "%s: null pointer", __func__);
    ANE_REQUIRE(x2 != x2norm, "%s: x2 and x2norm must be different buffers", __func__);
    ANE_REQUIRE(dtype_ok(dtype), "%s: bad dtype", __func__);
    if (int rc = check_bcs(__func__, B, C, S)) return rc;
    {
        const size_t nb = (size_t)B * C * S * dtype_size(dtype);
        ANE_CHECK_EXTENT(x2, nb); ANE_CHECK_EXTENT(x2norm, nb); ANE_CHECK_EXTENT(x, nb); ANE_CHECK_EXTENT(f, nb); ANE_CHECK_EXTENT(w, (size_t)C * 4);
    }
    ANE_DISPATCH_DTYPE(dtype, T, return (launch_rmsnorm_fwd<T, true>((cudaStream_t)stream, B, C, S, x2norm, x2, x, f, w, alpha, eps)));
    return ANE_CUDA_OK;
}

int ane_cuda_rmsnorm_bwd_dev(void *stream, ane_dtype dtype, int B, int C, int S, void *dx, float *dw, const void *dy,
                             const void *x, const float *w, const void *add, float eps, unsigned flags) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dx && dw && dy && x && w, "%s: null pointer", __func__);
    ANE_REQUIRE(dtype_ok(dtype), "%s: bad dtype", __func__);
    ANE_REQUIRE(flags == ANE_NORM_BWD_REFERENCE || flags == ANE_NORM_BWD_EXACT, "%s: bad flags %u", __func__, flags);
    if (int rc = check_bcs(__func__, B, C, S)) return rc;
    {
        const size_t nb = (size_t)B * C * S * dtype_size(dtype);
        ANE_CHECK_EXTENT(dx, nb); ANE_CHECK_EXTENT(dy, nb); ANE_CHECK_EXTENT(x, nb); ANE_CHECK_EXTENT(add, nb);
        ANE_CHECK_EXTENT(w, (size_t)C * 4); ANE_CHECK_EXTENT(dw, (size_t)C * 4);
    }
    return rmsnorm_bwd_any((cudaStream_t)stream, dtype, B, C, S, dx, dw, dy, x, w, add, eps, flags);
}

int ane_cuda_rmsnorm_bwd_static_dev(void *stream, ane_dtype dtype, int B, int C, int S, void *dx, float *dw, const void *dy,
                                    const void *x, const float *w, const void *add, float eps, unsigned flags) {
    // Deliberately independent of ane_cuda_init(): that call allocates, this path must not.
    ANE_REQUIRE(dx && dw && dy && x && w, "%s: null pointer", __func__);
    ANE_REQUIRE(dtype_ok(dtype), "%s: bad dtype", __func__);
    ANE_REQUIRE(flags == ANE_NORM_BWD_REFERENCE || flags == ANE_NORM_BWD_EXACT, "%s: bad flags %u", __func__, flags);
    ANE_REQUIRE(B >= 1 && C >= 1 && S >= 1, "%s: B, C, S must be positive (got %d, %d, %d)", __func__, B, C, S);
    if (C > STATIC_MAX_C)
        return fail(ANE_CUDA_ERR_UNSUPPORTED, "%s: C = %d exceeds the built-in scratch (at most %d channels); use ane_cuda_rmsnorm_bwd_dev",
                    __func__, C, STATIC_MAX_C);
    if ((long long)B * ((S + 7) / 8) > 0x7fffffffLL) return fail(ANE_CUDA_ERR_UNSUPPORTED, "%s: too many token tiles", __func__);
    float *partial = nullptr;
    int sms = 0;
    if (int rc = static_scratch_for_current_device(&partial, &sms)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // Nothing in the scratch has to start at zero: every block overwrites its whole row of
    // partials before the column sums read rows 0 .. grid-1, so leftovers of earlier calls are
    // never read.
    if (add) {
        ANE_DISPATCH_DTYPE(dtype, T, return (launch_rmsnorm_bwd_static<T, true>(st, partial, sms, B, C, S, dx, dw, dy, x, w, add, eps, flags)));
    } else {
        ANE_DISPATCH_DTYPE(dtype, T, return (launch_rmsnorm_bwd_static<T, false>(st, partial, sms, B, C, S, dx, dw, dy, x, w, nullptr, eps, flags)));
    }
    return ANE_CUDA_OK;
}

}  // extern "C"
