// norm_st.cuh -- shared-memory-resident RMSNorm kernels (single HBM pass, few registers).
//
// Measured on B200: a strided tile copy of a [B][C][S] tensor runs at 90-97 % of the flat copy
// rate as long as every block keeps its register count low enough for 3+ resident blocks per SM,
// even with row segments as narrow as 64 bytes (32-byte segments: 84-90 %).  These kernels are
// built to look like that copy: a block owns a [C x TB-byte] token strip, brings it into shared
// memory with asynchronous 16-byte copies (no register staging, the whole strip in flight at once),
// then sweeps the resident strip twice -- reduce, then normalise -- with one vector of state per
// thread.  Nothing is read twice from HBM or L2.
//   forward : strip of x (TB = 64 B per row, 64 KiB for C = 1024 in bf16), 3 blocks per SM
//   backward: strips of x and dy, the channels split over a pair of blocks (64-byte rows) or a cluster of four
//             (128-byte rows), 64 KiB per block for C = 1024 either way
#pragma once
#include "common.cuh"

#include <cooperative_groups.h>

#ifndef ANE_NORM_BWD_U
#define ANE_NORM_BWD_U 4
#endif
namespace ane {

namespace cgx = cooperative_groups;

constexpr int ST_THREADS = 256;

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// LG = 16-byte lanes per row segment (TB = 16*LG bytes), R = ST_THREADS/LG rows per step.
template <typename T, int LG, bool FUSE_RES>
__global__ void __launch_bounds__(ST_THREADS)
rmsnorm_fwd_st_kernel(T *out, T *x2out, const T *x, const T *f, const float *__restrict__ w, int C, int S,
                      int tiles_per_seq, float alpha, float eps) {
    constexpr int VEC = Elt<T>::VEC;
    constexpr int R = ST_THREADS / LG;
    constexpr int TW = LG * VEC;
    extern __shared__ uint4 strip[];                 // [C][LG]
    __shared__ __align__(16) float red[R][TW];
    __shared__ __align__(16) float tot[TW];

    const int b = blockIdx.x / tiles_per_seq;
    const int lg = threadIdx.x % LG, rg = threadIdx.x / LG;
    const int t = (blockIdx.x % tiles_per_seq) * TW + lg * VEC;
    const bool active = t < S;
    const size_t base = (size_t)b * C * S + t;
    dep_sync();

    if (active)
        for (int c = rg; c < C; c += R) cp_async16(&strip[c * LG + lg], x + base + (size_t)c * S);
    cp_async_commit();

    V<VEC> ss = V<VEC>::splat(0.0f);
    if (FUSE_RES) {
        // f streams through registers while x lands in shared memory; x2 replaces x in the strip
        constexpr int U = 4;
        cp_async_wait_all();        // this thread reads back only what it copied itself
        for (int cb = rg; cb < C; cb += R * U) {
            Raw<T, VEC> rf[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int c = cb + u * R;
                if (active && c < C) rf[u].load_stream(f + base + (size_t)c * S);
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int c = cb + u * R;
                if (active && c < C) {
                    Raw<T, VEC> rx;
                    rx.v = strip[c * LG + lg];
                    rx.put(vadd(vscale(rf[u].get(), alpha), rx.get()));           // train.m:460, two roundings
                    rx.store_stream(x2out + base + (size_t)c * S);
                    strip[c * LG + lg] = rx.v;
                    const V<VEC> v = rx.get();                                     // the stored (rounded) value
                    ss = vfma(v, v, ss);
                }
            }
        }
    } else {
        cp_async_wait_all();
        if (active) {
#pragma unroll 4
            for (int c = rg; c < C; c += R) {
                Raw<T, VEC> rx;
                rx.v = strip[c * LG + lg];
                const V<VEC> v = rx.get();
                ss = vfma(v, v, ss);
            }
        }
    }
    lanes_to_smem<VEC>(&red[rg][lg * VEC], ss);
    __syncthreads();
    {
        constexpr int P = ST_THREADS / TW;
        const float s = block_column_sum<R, TW, ST_THREADS>(&red[0][0], threadIdx.x);
        if (threadIdx.x % P == 0) tot[threadIdx.x / P] = 1.0f / sqrtf(__fadd_rn(__fmul_rn(s, 1.0f / (float)C), eps));
    }
    __syncthreads();
    if (!active) return;
    const V<VEC> rr = lanes_from_smem<VEC>(&tot[lg * VEC]);
#pragma unroll 4
    for (int c = rg; c < C; c += R) {
        Raw<T, VEC> rx;
        rx.v = strip[c * LG + lg];
        rx.put(vscale(vmul(rx.get(), rr), __ldg(w + c)));                          // stories_cpu_ops.h:16-19
        rx.store_stream(out + base + (size_t)c * S);
    }
}

// Backward on a PAIR of blocks (a thread-block cluster of two): the channels are split between the
// two blocks, so the x and dy strips of a 64-byte-wide token tile take C/2 * 128 bytes of shared
// memory per block (64 KiB for C = 1024: three blocks per SM) instead of C * 128.  Each block reduces
// its half of sum(x^2) and sum(dy*x*w) per token, the halves are exchanged through distributed
// shared memory behind one cluster barrier per tile, and both blocks finish their channels.  The
// pairs are persistent (pair i takes tiles i, i+pairs, ...) so dw leaves as one row per pair.
// Rows of 64 bytes, not 32: a 32-byte segment costs a 64-byte DRAM fetch.
template <typename T, int LG, bool HAS_ADD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(ST_THREADS, 3)
rmsnorm_bwd_pair_kernel(T *dx, float *__restrict__ partial, const T *dy, const T *x, const float *__restrict__ w,
                        const T *add, int C, int S, int tiles_per_seq, int ntiles, float eps, unsigned flags) {
    constexpr int VEC = Elt<T>::VEC;
    constexpr int R = ST_THREADS / LG;
    constexpr int TW = LG * VEC;
    constexpr int NW = ST_THREADS / 32;
    static_assert(TW <= ST_THREADS, "one thread per token for the exchange");
    extern __shared__ uint4 strip[];                 // x: [Cn][LG], dy: [Cn][LG], then dw accumulators float[Cn]
    __shared__ __align__(16) float red[2][NW][TW];
    __shared__ __align__(16) float tot[2][TW];
    __shared__ float xch[2][2][TW];                  // [tile parity][sum][token]: this block's halves, read by the peer

    cgx::cluster_group cluster = cgx::this_cluster();
    const unsigned rank = cluster.block_rank();
    const int half = (C + 1) / 2;
    const int c0 = (int)rank * half;
    const int Cn = (C - c0 < half ? C - c0 : half) > 0 ? (C - c0 < half ? C - c0 : half) : 0;
    uint4 *sx = strip, *sd = strip + (size_t)half * LG;
    float *dwacc = reinterpret_cast<float *>(strip + (size_t)2 * half * LG);
    const float *peer_xch = cluster.map_shared_rank(&xch[0][0][0], rank ^ 1u);

    const int lg = threadIdx.x % LG, rg = threadIdx.x / LG;
    const float invd = 1.0f / (float)C;
    const bool exact = (flags & ANE_NORM_BWD_EXACT) != 0;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

    for (int c = threadIdx.x; c < Cn; c += ST_THREADS) dwacc[c] = 0.0f;
    __syncthreads();
    dep_sync();

    // The strips are software-pipelined across tiles without any extra barrier: a strip entry is only ever touched
    // by the thread that copied it, so as soon as sweep 2 has read an entry the same thread issues the copy of the
    // NEXT tile's element into it.  By the end of sweep 2 the whole next tile is in flight.
    auto tile_base = [&](int tile, bool &act) -> size_t {
        const int b = tile / tiles_per_seq;
        const int t = (tile % tiles_per_seq) * TW + lg * VEC;
        act = t < S;
        return ((size_t)b * C + c0) * S + t;
    };
    {
        bool act0;
        const size_t base0 = pair < ntiles ? tile_base(pair, act0) : 0;
        if (pair < ntiles && act0)
            for (int c = rg; c < Cn; c += R) {
                cp_async16(&sx[c * LG + lg], x + base0 + (size_t)c * S);
                cp_async16(&sd[c * LG + lg], dy + base0 + (size_t)c * S);
            }
        cp_async_commit();
    }
    int it = 0;
    for (int tile = pair; tile < ntiles; tile += npairs, it ^= 1) {
        bool active, nactive = false;
        const size_t base = tile_base(tile, active);
        const bool has_next = tile + npairs < ntiles;
        const size_t nbase = has_next ? tile_base(tile + npairs, nactive) : 0;
        cp_async_wait_all();             // each thread reads back only what it copied itself

        V<VEC> ss = V<VEC>::splat(0.0f), dot = V<VEC>::splat(0.0f);
        if (active) {
#pragma unroll 4
            for (int c = rg; c < Cn; c += R) {
                Raw<T, VEC> rx, rd;
                rx.v = sx[c * LG + lg];
                rd.v = sd[c * LG + lg];
                const V<VEC> xv = rx.get(), dv = rd.get();
                ss = vfma(xv, xv, ss);
                dot = vfma_s(vmul(dv, xv), __ldg(w + c0 + c), dot);                // stories_cpu_ops.h:35-38
            }
        }
        ss = warp_rowgroup_sum<VEC, LG>(ss);
        dot = warp_rowgroup_sum<VEC, LG>(dot);
        if ((threadIdx.x & 31) < LG) {
            lanes_to_smem<VEC>(&red[0][threadIdx.x >> 5][lg * VEC], ss);
            lanes_to_smem<VEC>(&red[1][threadIdx.x >> 5][lg * VEC], dot);
        }
        __syncthreads();
        if (threadIdx.x < TW) {          // this block's halves, warps in fixed order
            float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
            for (int q = 0; q < NW; q++) { s0 += red[0][q][threadIdx.x]; s1 += red[1][q][threadIdx.x]; }
            xch[it][0][threadIdx.x] = s0;
            xch[it][1][threadIdx.x] = s1;
        }
        cluster.sync();                  // both halves published (also a block barrier)
        if (threadIdx.x < TW) {
            const float m0 = xch[it][0][threadIdx.x], m1 = xch[it][1][threadIdx.x];
            const float p0 = peer_xch[(it * 2 + 0) * TW + threadIdx.x], p1 = peer_xch[(it * 2 + 1) * TW + threadIdx.x];
            const float s0 = rank == 0 ? m0 + p0 : p0 + m0;        // lower channels first in both blocks: same bits
            const float s1 = rank == 0 ? m1 + p1 : p1 + m1;
            const float r1 = 1.0f / sqrtf(__fadd_rn(__fmul_rn(s0, invd), eps));
            float r2 = r1 * r1;
            r2 = r2 * invd;
            tot[0][threadIdx.x] = r1;
            tot[1][threadIdx.x] = s1 * r2;                                         // stories_cpu_ops.h:39-41
        }
        __syncthreads();
        const V<VEC> rr = lanes_from_smem<VEC>(&tot[0][lg * VEC]), coef = lanes_from_smem<VEC>(&tot[1][lg * VEC]);
        constexpr int U = 4;
        for (int cb = 0; cb < Cn; cb += R * U) {      // uniform trip count: the shuffles below need every lane
            Raw<T, VEC> ra[U];
            if (HAS_ADD) {
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int c = cb + u * R + rg;
                    if (active && c < Cn) ra[u].load_stream(add + base + (size_t)c * S);
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int c = cb + u * R + rg;
                float dwp = 0.0f;
                if (active && c < Cn) {
                    Raw<T, VEC> rx, rd;
                    rx.v = sx[c * LG + lg];
                    rd.v = sd[c * LG + lg];
                    const V<VEC> xv = rx.get(), dv = rd.get();
                    if (nactive) {       // this entry is free now: bring in the next tile's element
                        cp_async16(&sx[c * LG + lg], x + nbase + (size_t)c * S);
                        cp_async16(&sd[c * LG + lg], dy + nbase + (size_t)c * S);
                    }
                    const float wc = __ldg(w + c0 + c);
                    V<VEC> o;
                    if (exact) o = vmul(vsub(vscale(dv, wc), vmul(xv, coef)), rr);
                    else o = vscale(vmul(vsub(dv, vmul(xv, coef)), rr), wc);      // stories_cpu_ops.h:43-46
                    dwp = vmul(vmul(dv, xv), rr).hsum();                           // stories_cpu_ops.h:47-50
                    if (HAS_ADD) o = vadd(o, ra[u].get());                         // train.m:590,721
                    Raw<T, VEC> ro;
                    ro.put(o);
                    ro.store_stream(dx + base + (size_t)c * S);
                }
#pragma unroll
                for (int off = LG / 2; off > 0; off >>= 1) dwp += __shfl_xor_sync(0xffffffffu, dwp, off);
                if (lg == 0 && c < Cn) dwacc[c] += dwp;  // row group rg is the only writer of channel c
            }
        }
        if (!active && nactive) {        // this thread skipped sweep 2: issue its copies of the next tile here
            for (int c = rg; c < Cn; c += R) {
                cp_async16(&sx[c * LG + lg], x + nbase + (size_t)c * S);
                cp_async16(&sd[c * LG + lg], dy + nbase + (size_t)c * S);
            }
        }
        cp_async_commit();
        // red/tot/xch[it] are next written after the following tile's barriers, which every thread of the pair
        // reaches after this point
    }
    __syncthreads();
    for (int c = threadIdx.x; c < Cn; c += ST_THREADS) partial[(size_t)pair * C + c0 + c] = dwacc[c];
    cluster.sync();                      // the peer may still be reading xch
}

// Backward on a cluster of CL blocks, the general form of the pair kernel above.  The channels are split CL ways, so
// that a block can afford WIDER rows in the same shared memory: with CL = 4 the x and dy strips of a 128-byte-wide token
// tile take C/4 * 256 bytes (64 KiB for C = 1024, three blocks per SM), and a 128-byte row segment is a whole cache line
// where the pair kernel's 64-byte segment is half of one.  On B200 the row width is what this operator's speed follows.
// The CL partial sums per token cross through distributed shared memory behind one cluster barrier per tile and are
// added in block-rank order in every block (same bits everywhere).
//   NBUF = 1: one pair of strips; as in the pair kernel, sweep 2 refills each entry with the next tile's element.
//   NBUF = 2: two pairs of strips, the next tile is copied into the other pair before the current one is touched, so a
//             whole tile is in flight all the time (measured: no faster for 16-bit data, the fixed cost per tile of
//             the halved strips outweighs it).
// Strip entries are thread-owned (copied, read and recycled by one thread), so the copies need no barrier of their own.
__device__ __forceinline__ void cp_async_wait_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

template <typename T, int LG, bool HAS_ADD, int CL, int NBUF>
__global__ void __cluster_dims__(CL, 1, 1) __launch_bounds__(ST_THREADS, 3)
rmsnorm_bwd_cluster_kernel(T *dx, float *__restrict__ partial, const T *dy, const T *x, const float *__restrict__ w,
                        const T *add, int C, int S, int tiles_per_seq, int ntiles, float eps, unsigned flags) {
    constexpr int VEC = Elt<T>::VEC;
    constexpr int R = ST_THREADS / LG;
    constexpr int TW = LG * VEC;
    constexpr int NW = ST_THREADS / 32;
    constexpr int U = ANE_NORM_BWD_U;
    static_assert(TW <= ST_THREADS, "one thread per token for the exchange");
    extern __shared__ uint4 strip[];                 // [NBUF buffers][x: [part][LG], dy: [part][LG]], then dw accumulators float[part]
    __shared__ __align__(16) float red[2][NW][TW];
    __shared__ __align__(16) float tot[2][TW];
    __shared__ float xch[2][2][TW];                  // [tile parity][sum][token]: this block's part, read by the peers

    cgx::cluster_group cluster = cgx::this_cluster();
    const unsigned rank = cluster.block_rank();
    const int part = (C + CL - 1) / CL;
    const int c0 = (int)rank * part;
    const int Cn = C - c0 < part ? (C - c0 > 0 ? C - c0 : 0) : part;
    float *dwacc = reinterpret_cast<float *>(strip + (size_t)2 * NBUF * part * LG);

    const int lg = threadIdx.x % LG, rg = threadIdx.x / LG;
    const float invd = 1.0f / (float)C;
    const bool exact = (flags & ANE_NORM_BWD_EXACT) != 0;
    const int group = blockIdx.x / CL, ngroups = gridDim.x / CL;

    for (int c = threadIdx.x; c < Cn; c += ST_THREADS) dwacc[c] = 0.0f;
    __syncthreads();
    dep_sync();

    auto tile_base = [&](int tile, bool &act) -> size_t {
        const int b = tile / tiles_per_seq;
        const int t = (tile % tiles_per_seq) * TW + lg * VEC;
        act = t < S;
        return ((size_t)b * C + c0) * S + t;
    };
    auto copy_in = [&](int tile, int buf) {           // this thread's entries of one tile; always closes a copy group
        if (tile < ntiles) {
            bool act;
            const size_t base = tile_base(tile, act);
            uint4 *sx = strip + (size_t)buf * 2 * part * LG, *sd = sx + (size_t)part * LG;
            if (act)
                for (int c = rg; c < Cn; c += R) {
                    cp_async16(&sx[c * LG + lg], x + base + (size_t)c * S);
                    cp_async16(&sd[c * LG + lg], dy + base + (size_t)c * S);
                }
        }
        cp_async_commit();
    };
    copy_in(group, 0);
    int it = 0;
    for (int tile = group; tile < ntiles; tile += ngroups, it ^= 1) {
        bool active;
        const size_t base = tile_base(tile, active);
        uint4 *sx = strip + (size_t)(it & (NBUF - 1)) * 2 * part * LG, *sd = sx + (size_t)part * LG;
        bool nactive = false;             // NBUF == 1: the next tile is copied in entry by entry during sweep 2
        const size_t nbase = tile + ngroups < ntiles ? tile_base(tile + ngroups, nactive) : 0;
        if (NBUF == 2) copy_in(tile + ngroups, it ^ 1);  // the other buffer was last read by this thread in the previous tile's sweep 2
        if (NBUF == 2) cp_async_wait_but_one();          // this tile has landed; each thread reads back only what it copied itself
        else cp_async_wait_all();

        V<VEC> ss = V<VEC>::splat(0.0f), dot = V<VEC>::splat(0.0f);
        if (active) {
#pragma unroll 4
            for (int c = rg; c < Cn; c += R) {
                Raw<T, VEC> rx, rd;
                rx.v = sx[c * LG + lg];
                rd.v = sd[c * LG + lg];
                const V<VEC> xv = rx.get(), dv = rd.get();
                ss = vfma(xv, xv, ss);
                dot = vfma_s(vmul(dv, xv), __ldg(w + c0 + c), dot);                // stories_cpu_ops.h:35-38
            }
        }
        ss = warp_rowgroup_sum<VEC, LG>(ss);
        dot = warp_rowgroup_sum<VEC, LG>(dot);
        if ((threadIdx.x & 31) < LG) {
            lanes_to_smem<VEC>(&red[0][threadIdx.x >> 5][lg * VEC], ss);
            lanes_to_smem<VEC>(&red[1][threadIdx.x >> 5][lg * VEC], dot);
        }
        __syncthreads();
        if (threadIdx.x < TW) {          // this block's part, warps in fixed order
            float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
            for (int q = 0; q < NW; q++) { s0 += red[0][q][threadIdx.x]; s1 += red[1][q][threadIdx.x]; }
            xch[it][0][threadIdx.x] = s0;
            xch[it][1][threadIdx.x] = s1;
        }
        cluster.sync();                  // every part published (also a block barrier)
        if (threadIdx.x < TW) {
            float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
            for (int q = 0; q < CL; q++) {                                          // lower channels first in every block
                const float *px = cluster.map_shared_rank(&xch[0][0][0], (unsigned)q);
                s0 += px[(it * 2 + 0) * TW + threadIdx.x];
                s1 += px[(it * 2 + 1) * TW + threadIdx.x];
            }
            const float r1 = 1.0f / sqrtf(__fadd_rn(__fmul_rn(s0, invd), eps));
            float r2 = r1 * r1;
            r2 = r2 * invd;
            tot[0][threadIdx.x] = r1;
            tot[1][threadIdx.x] = s1 * r2;                                         // stories_cpu_ops.h:39-41
        }
        __syncthreads();
        const V<VEC> rr = lanes_from_smem<VEC>(&tot[0][lg * VEC]), coef = lanes_from_smem<VEC>(&tot[1][lg * VEC]);
        for (int cb = 0; cb < Cn; cb += R * U) {      // uniform trip count: the shuffles below need every lane
            Raw<T, VEC> rb[U];
            if (HAS_ADD) {
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int c = cb + u * R + rg;
                    if (active && c < Cn) rb[u].load_stream(add + base + (size_t)c * S);
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int c = cb + u * R + rg;
                float dwp = 0.0f;
                if (active && c < Cn) {
                    Raw<T, VEC> rx, rd;
                    rx.v = sx[c * LG + lg];
                    rd.v = sd[c * LG + lg];
                    const V<VEC> xv = rx.get(), dv = rd.get();
                    if (NBUF == 1 && nactive) {  // this entry is free now: bring in the next tile's element
                        cp_async16(&sx[c * LG + lg], x + nbase + (size_t)c * S);
                        cp_async16(&sd[c * LG + lg], dy + nbase + (size_t)c * S);
                    }
                    const float wc = __ldg(w + c0 + c);
                    V<VEC> o;
                    if (exact) o = vmul(vsub(vscale(dv, wc), vmul(xv, coef)), rr);
                    else o = vscale(vmul(vsub(dv, vmul(xv, coef)), rr), wc);      // stories_cpu_ops.h:43-46
                    dwp = vmul(vmul(dv, xv), rr).hsum();                           // stories_cpu_ops.h:47-50
                    if (HAS_ADD) o = vadd(o, rb[u].get());                         // train.m:590,721
                    Raw<T, VEC> ro;
                    ro.put(o);
                    ro.store_stream(dx + base + (size_t)c * S);
                }
#pragma unroll
                for (int off = LG / 2; off > 0; off >>= 1) dwp += __shfl_xor_sync(0xffffffffu, dwp, off);
                if (lg == 0 && c < Cn) dwacc[c] += dwp;  // row group rg is the only writer of channel c
            }
        }
        if (NBUF == 1) {
            if (!active && nactive) {    // this thread skipped sweep 2: issue its copies of the next tile here
                for (int c = rg; c < Cn; c += R) {
                    cp_async16(&sx[c * LG + lg], x + nbase + (size_t)c * S);
                    cp_async16(&sd[c * LG + lg], dy + nbase + (size_t)c * S);
                }
            }
            cp_async_commit();
        }
        // red/tot/xch[it] are next written after the following tile's barriers, which every thread of the cluster
        // reaches after this point
    }
    cp_async_wait_all();
    __syncthreads();
    for (int c = threadIdx.x; c < Cn; c += ST_THREADS) partial[(size_t)group * C + c0 + c] = dwacc[c];
    cluster.sync();                      // a peer may still be reading xch
}

}  // namespace ane
