// xent.cu -- classifier softmax cross-entropy, forward and backward in one operator, over
// channel-first fp32 logits [B][V][S] (training/stories_cpu_ops.h:71-108,
// training/training_dynamic/cpu_ops.h:68-93).
//
// Per token t: m = max_v l, e = exp(l - m), p = e / sum e, loss_t = -log(p[tgt] + 1e-10),
// dlogits = (p - onehot) * (1/S) * grad_scale.  The reduction runs over V with stride S.
//
// A block owns a stripe of LG*4 tokens (128 bytes per vocabulary row) and sweeps the V rows
// twice: an online (max, sum) pass, then the pass that writes dlogits.  Loss terms go to a
// per-token scratch array and are summed per sequence in a fixed order by a second kernel.
#include "common.cuh"

#include <cooperative_groups.h>
#include <math.h>

namespace cg = cooperative_groups;

namespace ane {

constexpr int XE_THREADS = 256;
constexpr int XE_U = 4;

// exp(x) on the special-function unit: 2^(x*log2(e)), relative error about 2^-22 plus the rounding of
// the scaled argument -- below 2e-6 for |x| < 40, inside the 1e-5 contract.  The accurate expf costs
// ~20 instructions per element, which made this operator issue-bound instead of memory-bound.
constexpr float XC_LOG2E = 1.4426950408889634f;
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}


// CL > 1: the kernel is launched in clusters of CL blocks that share a stripe; block r of a cluster sweeps the
// vocabulary rows [r * rows_per_block, (r + 1) * rows_per_block) and the CL (max, sum) pairs per token cross through
// distributed shared memory once, between the sweeps.  It keeps every SM busy when there are few stripes.
template <typename ID, int VEC, int LG, int CL>
__global__ void __launch_bounds__(XE_THREADS)
xent_kernel(float *dlogits, const float *logits, const void *__restrict__ targets, float *__restrict__ loss_tok,
            int V, int S, int tiles_per_seq, int rows_per_block, float grad_scale, ane_cuda_status *status, int reverse) {
    constexpr int R = XE_THREADS / LG;
    constexpr int TW = LG * VEC;
    __shared__ float red_m[R][TW];
    __shared__ float red_s[R][TW];
    __shared__ float tot_m[TW];
    __shared__ float tot_is[TW];
    __shared__ float xpart[2][TW];       // CL > 1: this block's (max, sum) per token, read by the other blocks of the cluster

    const int stripe = blockIdx.x / CL, crank = blockIdx.x % CL;      // clusters are consecutive blocks
    const int v0 = CL > 1 ? crank * rows_per_block : 0;
    const int v1 = CL > 1 ? (v0 + rows_per_block < V ? v0 + rows_per_block : V) : V;
    const int b = stripe / tiles_per_seq;
    const int lg = threadIdx.x % LG, rg = threadIdx.x / LG;
    const int t = (stripe % tiles_per_seq) * TW + lg * VEC;
    const bool active = t < S;
    const size_t base = (size_t)b * V * S + t;

    // sweep 1: online max / sum of exp
    float m[VEC], s[VEC];
#pragma unroll
    for (int j = 0; j < VEC; j++) { m[j] = -INFINITY; s[j] = 0.0f; }
    for (int vb = v0; vb < v1; vb += R * XE_U) {
        Raw<float, VEC> r[XE_U];
        bool ok[XE_U];
#pragma unroll
        for (int u = 0; u < XE_U; u++) {
            const int v = vb + u * R + rg;
            ok[u] = active && v < v1;
            if (ok[u]) r[u].load(logits + base + (size_t)v * S);
        }
        float l[XE_U][VEC];
        float gm[VEC];
#pragma unroll
        for (int j = 0; j < VEC; j++) gm[j] = m[j];
#pragma unroll
        for (int u = 0; u < XE_U; u++) {
            if (ok[u]) {
                r[u].unpack(l[u]);
#pragma unroll
                for (int j = 0; j < VEC; j++) gm[j] = fmaxf(gm[j], l[u][j]);
            }
        }
#pragma unroll
        for (int j = 0; j < VEC; j++) {
            if (gm[j] > m[j]) { s[j] = s[j] * ex2_approx((m[j] - gm[j]) * XC_LOG2E); m[j] = gm[j]; }   // 2^-inf = 0 on the first group
        }
#pragma unroll
        for (int u = 0; u < XE_U; u++) {
            if (ok[u]) {
#pragma unroll
                for (int j = 0; j < VEC; j++) s[j] += ex2_approx(fmaf(l[u][j], XC_LOG2E, -m[j] * XC_LOG2E));
            }
        }
    }
#pragma unroll
    for (int j = 0; j < VEC; j++) { red_m[rg][lg * VEC + j] = m[j]; red_s[rg][lg * VEC + j] = s[j]; }
    __syncthreads();
    if (threadIdx.x < TW) {
        float M = -INFINITY;
        for (int q = 0; q < R; q++) M = fmaxf(M, red_m[q][threadIdx.x]);
        float sum = 0.0f;
        for (int q = 0; q < R; q++) {
            const float mq = red_m[q][threadIdx.x];
            if (mq > -INFINITY) sum += red_s[q][threadIdx.x] * expf(mq - M);
        }
        if (CL == 1) {
            tot_m[threadIdx.x] = M;
            tot_is[threadIdx.x] = 1.0f / sum;                // inv_sum, stories_cpu_ops.h:91-92
        } else {
            xpart[0][threadIdx.x] = M;
            xpart[1][threadIdx.x] = sum;
        }
    }
    if constexpr (CL > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();                                      // every block's pair is published (also a block barrier)
        if (threadIdx.x < TW) {                              // the same merge, in block order, in every block
            float pm[CL], ps[CL];
            float M = -INFINITY;
#pragma unroll
            for (int q = 0; q < CL; q++) {
                const float *px = cluster.map_shared_rank(&xpart[0][0], (unsigned)q);
                pm[q] = px[threadIdx.x];
                ps[q] = px[TW + threadIdx.x];
                M = fmaxf(M, pm[q]);
            }
            float sum = 0.0f;
#pragma unroll
            for (int q = 0; q < CL; q++)
                if (pm[q] > -INFINITY) sum += ps[q] * expf(pm[q] - M);
            tot_m[threadIdx.x] = M;
            tot_is[threadIdx.x] = 1.0f / sum;
        }
    }
    __syncthreads();

    float negML[VEC], inv[VEC], scale[VEC];
    int tgt[VEC];
    const float invS = 1.0f / (float)S;
#pragma unroll
    for (int j = 0; j < VEC; j++) {
        negML[j] = -tot_m[lg * VEC + j] * XC_LOG2E;
        inv[j] = tot_is[lg * VEC + j];
        tgt[j] = -1;
        if (active) {
            const int id = (int)reinterpret_cast<const ID *>(targets)[(size_t)b * S + t + j];
            if (id >= 0 && id < V) tgt[j] = id;
            else if (rg == 0 && crank == 0) {                  // one thread per token reports it
                atomicAdd(&status->oor_ids, 1);
                loss_tok[(size_t)b * S + t + j] = 0.0f;        // no loss term (stories_cpu_ops.h:98)
            }
        }
        float sc = inv[j];
        if (tgt[j] >= 0) sc = sc * invS;                       // an out-of-range target keeps the plain softmax
        if (grad_scale != 1.0f) sc = sc * grad_scale;
        scale[j] = sc;
    }

    // sweep 2: p = exp(l - M) * inv_sum ; target row: loss and -1 ; then *1/S (and grad_scale).  `reverse`: the row groups are
    // walked from the last one down, so the rows sweep 1 read last -- the ones most likely still in L2 -- are read first
    // (every element is computed on its own: the direction does not change a bit of the result).
    const int ngroups = v1 > v0 ? (v1 - v0 + R * XE_U - 1) / (R * XE_U) : 0;
    for (int gi = 0; gi < ngroups; gi++) {
        const int vb = v0 + (reverse ? ngroups - 1 - gi : gi) * (R * XE_U);
        Raw<float, VEC> r[XE_U];
        bool ok[XE_U];
#pragma unroll
        for (int u = 0; u < XE_U; u++) {
            const int v = vb + u * R + rg;
            ok[u] = active && v < v1;
            if (ok[u]) r[u].load_stream(logits + base + (size_t)v * S);
        }
#pragma unroll
        for (int u = 0; u < XE_U; u++) {
            const int v = vb + u * R + rg;
            if (ok[u]) {
                float l[VEC];
                r[u].unpack(l);
#pragma unroll
                for (int j = 0; j < VEC; j++) {
                    const float e = ex2_approx(fmaf(l[j], XC_LOG2E, negML[j]));
                    float p = e * scale[j];
                    if (v == tgt[j]) {
                        const float pr = e * inv[j];
                        const float lt = -logf(pr + 1e-10f);                       // stories_cpu_ops.h:99
                        loss_tok[(size_t)b * S + t + j] = lt;
                        if (!isfinite(lt)) atomicAdd(&status->nonfinite, 1);
                        p = (pr - 1.0f) * invS;
                        if (grad_scale != 1.0f) p = p * grad_scale;
                    }
                    l[j] = p;
                }
                Raw<float, VEC> o;
                o.pack(l);
                o.store_stream(dlogits + base + (size_t)v * S);
            }
        }
    }
    if constexpr (CL > 1) cg::this_cluster().sync();         // a peer may still be reading xpart
}

// ------------------------------------------------------------------ cluster kernel
// One token's column is V*4 bytes (152 KB for V = 37984, 608 KB for V = 151936): a block cannot keep
// its stripe on chip, and with one block per stripe the whole GPU has hundreds of stripes (GBs) in
// flight, so the second sweep always comes from HBM again (3 bytes moved per 2 needed).
// Here a thread-block CLUSTER of XC_CL blocks owns a 16-token stripe (64-byte rows); block r of the
// cluster takes vocabulary rows [r*rows_per_cta, (r+1)*rows_per_cta):
//   1. the first `rows_res` rows of the slice are copied into shared memory with asynchronous 16-byte
//      copies (up to 192 KB per SM in flight, no register staging), every entry by the thread that
//      will use it; the rows that do not fit (if any) stream through registers meanwhile;
//   2. online (max, sum) per token over the slice; warp shuffles, then shared memory, give the
//      block's pair; the cluster exchanges the XC_CL pairs through distributed shared memory
//      (hardware cluster barrier -- no flags in global memory, no cooperative launch);
//   3. the slice is swept again FROM SHARED MEMORY to write dlogits; only the non-resident rows
//      are read a second time (from L2 when the slices in flight fit there).
// With V = 37984 about two thirds of every slice never leaves the SM between the sweeps.
constexpr int XC_CL = 8;               // blocks per cluster (portable maximum)
constexpr int XC_LG = 4;               // 16-byte lanes per row: 16 tokens, 64-byte rows
constexpr int XC_TW = XC_LG * 4;
constexpr int XC_UNIT = 256;           // resident rows are budgeted in units of 256 rows (16 KB)
constexpr int XC_MAXUNITS = 12;        // 192 KB per block
constexpr int XC_U = 4;

// running (max, sum) of four tokens; ml = max * log2(e)
struct Ms4 { float m[4], s[4]; };

__device__ __forceinline__ void ms_init(Ms4 &a) {
#pragma unroll
    for (int j = 0; j < 4; j++) { a.m[j] = -INFINITY; a.s[j] = 0.0f; }
}
__device__ __forceinline__ void ms_raise(Ms4 &a, const float (&gm)[4]) {
#pragma unroll
    for (int j = 0; j < 4; j++)
        if (gm[j] > a.m[j]) { a.s[j] = a.s[j] * ex2_approx((a.m[j] - gm[j]) * XC_LOG2E); a.m[j] = gm[j]; }   // 2^-inf = 0 the first time
}
// fold U rows (held as float4) into the running (max, sum): one rescale per group
template <int U>
__device__ __forceinline__ void ms_fold(Ms4 &a, const float4 (&r)[U], const bool (&ok)[U]) {
    float gm[4] = {a.m[0], a.m[1], a.m[2], a.m[3]};
#pragma unroll
    for (int u = 0; u < U; u++)
        if (ok[u]) {
            gm[0] = fmaxf(gm[0], r[u].x); gm[1] = fmaxf(gm[1], r[u].y);
            gm[2] = fmaxf(gm[2], r[u].z); gm[3] = fmaxf(gm[3], r[u].w);
        }
    ms_raise(a, gm);
    const float n0 = -a.m[0] * XC_LOG2E, n1 = -a.m[1] * XC_LOG2E, n2 = -a.m[2] * XC_LOG2E, n3 = -a.m[3] * XC_LOG2E;
#pragma unroll
    for (int u = 0; u < U; u++)
        if (ok[u]) {
            a.s[0] += ex2_approx(fmaf(r[u].x, XC_LOG2E, n0)); a.s[1] += ex2_approx(fmaf(r[u].y, XC_LOG2E, n1));
            a.s[2] += ex2_approx(fmaf(r[u].z, XC_LOG2E, n2)); a.s[3] += ex2_approx(fmaf(r[u].w, XC_LOG2E, n3));
        }
}
__device__ __forceinline__ void ms_merge(float &m, float &s, float m2, float s2) {
    const float M = fmaxf(m, m2);
    float acc = 0.0f;
    if (m > -INFINITY) acc += s * expf(m - M);
    if (m2 > -INFINITY) acc += s2 * expf(m2 - M);
    m = M;
    s = acc;
}

// Per-thread constants of the second sweep.  p = softmax probability of a row; the row that is a
// token's target takes the slow path (stories_cpu_ops.h:97-103).
struct XentRowOut {
    float scale[4];       // (1/sum) * (1/S) * grad_scale   (out-of-range target: no 1/S, stories_cpu_ops.h:98)
    float inv[4];         // 1/sum
    int tgt[4];
    float invS, grad_scale;
    float *loss_tok;      // already offset to this thread's first token
    ane_cuda_status *status;
};
// e[j] = exp(l - M) (or exp(l - m_t) with the difference folded into scale/inv); v = vocabulary row
__device__ __forceinline__ float4 xent_finish(const float (&e)[4], int v, const XentRowOut &o) {
    float p[4];
#pragma unroll
    for (int j = 0; j < 4; j++) p[j] = e[j] * o.scale[j];
    if (v == o.tgt[0] || v == o.tgt[1] || v == o.tgt[2] || v == o.tgt[3]) {
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (v == o.tgt[j]) {
                const float pr = e[j] * o.inv[j];
                const float lt = -logf(pr + 1e-10f);                                // stories_cpu_ops.h:99
                o.loss_tok[j] = lt;
                if (!isfinite(lt)) atomicAdd(&o.status->nonfinite, 1);
                float q = (pr - 1.0f) * o.invS;
                if (o.grad_scale != 1.0f) q = q * o.grad_scale;
                p[j] = q;
            }
    }
    return make_float4(p[0], p[1], p[2], p[3]);
}

__device__ __forceinline__ void xc_cp_async16(void *smem_dst, const void *gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void xc_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void xc_cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Persistent clusters: cluster i takes stripes i, i + clusters, ...  The resident part of a block's slice is an
// array of 16-byte entries, each touched by ONE thread only (it copies the entry in, sweeps it three times, and
// -- as soon as the last sweep has read it -- copies the NEXT stripe's element into it), so the stripes are
// software-pipelined without any barrier beyond the one cluster barrier per stripe.
template <typename ID, int THREADS>
__global__ void __cluster_dims__(XC_CL, 1, 1) __launch_bounds__(THREADS, 1024 / THREADS)
xent_cluster_kernel(float *dlogits, const float *logits, const void *__restrict__ targets, float *__restrict__ loss_tok,
                    int V, int S, int stripes_per_seq, int nstripes, int rows_per_cta, int rows_res, float grad_scale,
                    ane_cuda_status *status) {
    constexpr int R = THREADS / XC_LG;
    constexpr int NW = THREADS / 32;
    extern __shared__ uint8_t xc_raw[];
    __shared__ float2 red[NW][XC_TW];
    __shared__ float2 part[2][XC_TW];     // [stripe parity]: this block's (max, sum) per token; peers read it
    __shared__ float2 fin[XC_TW];         // (max, 1/sum) over the whole vocabulary

    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank();
    float4 *res = reinterpret_cast<float4 *>((reinterpret_cast<uintptr_t>(xc_raw) + 127) & ~(uintptr_t)127);   // [rows][XC_LG]

    const int lg = threadIdx.x % XC_LG, rg = threadIdx.x / XC_LG;
    const int v0 = (int)rank * rows_per_cta;
    const int v1 = v0 + rows_per_cta < V ? v0 + rows_per_cta : V;
    const int rows = v1 > v0 ? v1 - v0 : 0;
    const int nres = rows < rows_res ? rows : rows_res;
    const int cid = blockIdx.x / XC_CL, ncl = gridDim.x / XC_CL;

    auto stripe_base = [&](int stripe, bool &act, int &b, int &t) -> size_t {
        b = stripe / stripes_per_seq;
        t = (stripe % stripes_per_seq) * XC_TW + lg * 4;
        act = t < S;
        return (size_t)b * V * S + t;
    };
    {   // first stripe's resident rows
        bool act;
        int b, t;
        if (cid < nstripes) {
            const size_t base0 = stripe_base(cid, act, b, t);
            if (act)
                for (int q = rg; q < nres; q += R) xc_cp_async16(&res[q * XC_LG + lg], logits + base0 + (size_t)(v0 + q) * S);
        }
        xc_cp_async_commit();
    }

    int par = 0;
    for (int stripe = cid; stripe < nstripes; stripe += ncl, par ^= 1) {
        bool active, nactive = false;
        int b, t, nb, nt;
        const size_t base = stripe_base(stripe, active, b, t);
        const bool has_next = stripe + ncl < nstripes;
        const size_t nbase = has_next ? stripe_base(stripe + ncl, nactive, nb, nt) : 0;

        // ---- sweep 1a: rows that do not fit in shared memory, through registers (they stay in L2)
        Ms4 ms;
        ms_init(ms);
        for (int vb = v0 + nres; vb < v1; vb += R * XC_U) {
            float4 r[XC_U];
            bool ok[XC_U];
#pragma unroll
            for (int u = 0; u < XC_U; u++) {
                const int v = vb + u * R + rg;
                ok[u] = active && v < v1;
                if (ok[u]) r[u] = *reinterpret_cast<const float4 *>(logits + base + (size_t)v * S);
            }
            ms_fold<XC_U>(ms, r, ok);
        }
        xc_cp_async_wait_all();           // this thread's resident entries have landed
        // ---- sweep 1b: maximum over this thread's resident rows
        float gm[4] = {ms.m[0], ms.m[1], ms.m[2], ms.m[3]};
        if (active) {
#pragma unroll 4
            for (int q = rg; q < nres; q += R) {
                const float4 r = res[q * XC_LG + lg];
                gm[0] = fmaxf(gm[0], r.x); gm[1] = fmaxf(gm[1], r.y); gm[2] = fmaxf(gm[2], r.z); gm[3] = fmaxf(gm[3], r.w);
            }
        }
        ms_raise(ms, gm);
        // ---- sweep 1c: e = exp(l - m_thread) replaces l in shared memory; the sum accumulates
        if (active) {
            const float n0 = -ms.m[0] * XC_LOG2E, n1 = -ms.m[1] * XC_LOG2E, n2 = -ms.m[2] * XC_LOG2E, n3 = -ms.m[3] * XC_LOG2E;
#pragma unroll 4
            for (int q = rg; q < nres; q += R) {
                float4 r = res[q * XC_LG + lg];
                r.x = ex2_approx(fmaf(r.x, XC_LOG2E, n0)); r.y = ex2_approx(fmaf(r.y, XC_LOG2E, n1));
                r.z = ex2_approx(fmaf(r.z, XC_LOG2E, n2)); r.w = ex2_approx(fmaf(r.w, XC_LOG2E, n3));
                ms.s[0] += r.x; ms.s[1] += r.y; ms.s[2] += r.z; ms.s[3] += r.w;
                res[q * XC_LG + lg] = r;
            }
        }
        const float mt[4] = {ms.m[0], ms.m[1], ms.m[2], ms.m[3]};      // the reference point of this thread's e values

        // ---- block (max, sum): row groups of a warp by shuffles, warps through shared memory
#pragma unroll
        for (int off = XC_LG; off < 32; off <<= 1) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float m2 = __shfl_xor_sync(0xffffffffu, ms.m[j], off);
                const float s2 = __shfl_xor_sync(0xffffffffu, ms.s[j], off);
                ms_merge(ms.m[j], ms.s[j], m2, s2);
            }
        }
        if ((threadIdx.x & 31) < XC_LG) {
#pragma unroll
            for (int j = 0; j < 4; j++) red[threadIdx.x >> 5][lg * 4 + j] = make_float2(ms.m[j], ms.s[j]);
        }
        __syncthreads();
        if (threadIdx.x < XC_TW) {
            float m = -INFINITY, s = 0.0f;
            for (int q = 0; q < NW; q++) ms_merge(m, s, red[q][threadIdx.x].x, red[q][threadIdx.x].y);
            part[par][threadIdx.x] = make_float2(m, s);
        }
        cluster.sync();                                   // every block's pair is published (also a block barrier)
        if (threadIdx.x < XC_TW) {
            float m = -INFINITY, s = 0.0f;
            for (unsigned q = 0; q < XC_CL; q++) {        // fixed rank order: all blocks get the same bits
                const float2 pq = cluster.map_shared_rank(&part[0][0], q)[par * XC_TW + threadIdx.x];
                ms_merge(m, s, pq.x, pq.y);
            }
            fin[threadIdx.x] = make_float2(m, 1.0f / s);                                 // inv_sum, stories_cpu_ops.h:91-92
        }
        __syncthreads();
        // part[par] is written again two stripes later, after the next stripe's cluster barrier, which every block
        // reaches only after these reads; fin and red are rewritten after this stripe's sweep 2 (barriers above).

        XentRowOut o;
        float negML[4], rel[4];
        o.invS = 1.0f / (float)S;
        o.grad_scale = grad_scale;
        o.status = status;
        o.loss_tok = loss_tok + (size_t)b * S + t;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 f = fin[lg * 4 + j];
            negML[j] = -f.x * XC_LOG2E;
            rel[j] = mt[j] > -INFINITY ? ex2_approx((mt[j] - f.x) * XC_LOG2E) : 0.0f;   // exp(m_thread - M)
            o.inv[j] = f.y;
            o.tgt[j] = -1;
            if (active) {
                const int id = (int)reinterpret_cast<const ID *>(targets)[(size_t)b * S + t + j];
                if (id >= 0 && id < V) o.tgt[j] = id;
                else if (rg == 0 && rank == 0) {                  // one thread per token reports it
                    atomicAdd(&status->oor_ids, 1);
                    o.loss_tok[j] = 0.0f;                         // no loss term (stories_cpu_ops.h:98)
                }
            }
            float sc = o.inv[j];
            if (o.tgt[j] >= 0) sc = sc * o.invS;
            if (grad_scale != 1.0f) sc = sc * grad_scale;
            o.scale[j] = sc;
        }
        // ---- sweep 2a: non-resident rows again (read first: they were touched longest ago)
        for (int vb = v0 + nres; vb < v1; vb += R * XC_U) {
            float4 r[XC_U];
            bool ok[XC_U];
#pragma unroll
            for (int u = 0; u < XC_U; u++) {
                const int v = vb + u * R + rg;
                ok[u] = active && v < v1;
                if (ok[u]) r[u] = __ldcs(reinterpret_cast<const float4 *>(logits + base + (size_t)v * S));
            }
#pragma unroll
            for (int u = 0; u < XC_U; u++) {
                const int v = vb + u * R + rg;
                if (ok[u]) {
                    const float e[4] = {ex2_approx(fmaf(r[u].x, XC_LOG2E, negML[0])), ex2_approx(fmaf(r[u].y, XC_LOG2E, negML[1])),
                                        ex2_approx(fmaf(r[u].z, XC_LOG2E, negML[2])), ex2_approx(fmaf(r[u].w, XC_LOG2E, negML[3]))};
                    __stcs(reinterpret_cast<float4 *>(dlogits + base + (size_t)v * S), xent_finish(e, v, o));
                }
            }
        }
        // ---- sweep 2b: resident rows from shared memory (e values relative to this thread's maximum); every entry
        // is refilled with the next stripe's element as soon as it has been read
        if (active) {
#pragma unroll
            for (int j = 0; j < 4; j++) { o.scale[j] *= rel[j]; o.inv[j] *= rel[j]; }
#pragma unroll 4
            for (int q = rg; q < nres; q += R) {
                const float4 r = res[q * XC_LG + lg];
                const float e[4] = {r.x, r.y, r.z, r.w};
                if (nactive) xc_cp_async16(&res[q * XC_LG + lg], logits + nbase + (size_t)(v0 + q) * S);
                __stcs(reinterpret_cast<float4 *>(dlogits + base + (size_t)(v0 + q) * S), xent_finish(e, v0 + q, o));
            }
        } else if (nactive) {
            for (int q = rg; q < nres; q += R) xc_cp_async16(&res[q * XC_LG + lg], logits + nbase + (size_t)(v0 + q) * S);
        }
        xc_cp_async_commit();
    }
    cluster.sync();                                       // peers may still be reading `part`
}

// loss_seq[b] = (sum_t loss_tok[b][t]) / S, fixed summation tree.
__global__ void __launch_bounds__(256) xent_loss_kernel(float *__restrict__ loss_seq, const float *__restrict__ loss_tok, int S) {
    __shared__ float sh[8];
    const float *p = loss_tok + (size_t)blockIdx.x * S;
    float acc = 0.0f;
    for (int t = threadIdx.x; t < S; t += 256) acc += p[t];
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int i = 0; i < 8; i++) s += sh[i];
        loss_seq[blockIdx.x] = s / (float)S;
    }
}

}  // namespace ane

using namespace ane;

// One block per stripe of LG * VEC tokens, or -- when that leaves SMs idle -- a cluster of CL blocks per stripe.
template <typename ID, int VEC, int LG, int CL>
static int launch_xent_cl(cudaStream_t st, unsigned nstripes, int V, int S, int tps, float *dlogits, const float *logits,
                          const void *targets, float *loss_tok, float grad_scale, ane_cuda_status *status) {
    const int rows_per_block = (V + CL - 1) / CL;
    // second sweep from the last row group down (measured: 0.642 / 0.648 / 0.647 of the copy rate for V = 151936 / 37984 /
    // 9200 against 0.634 / 0.641 / 0.636 in the forward direction: what sweep 1 read last is still in L2)
    const int reverse = tuning("xent_reverse", 1);
    if (CL == 1) {
        xent_kernel<ID, VEC, LG, CL><<<nstripes, XE_THREADS, 0, st>>>(dlogits, logits, targets, loss_tok, V, S, tps, rows_per_block, grad_scale, status, reverse);
        return ANE_CUDA_OK;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(nstripes * CL, 1, 1);
    cfg.blockDim = dim3(XE_THREADS, 1, 1);
    cfg.stream = st;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = CL; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    ANE_CUDA_TRY(cudaLaunchKernelEx(&cfg, xent_kernel<ID, VEC, LG, CL>, dlogits, logits, targets, loss_tok, V, S, tps, rows_per_block, grad_scale, status, reverse));
    return ANE_CUDA_OK;
}

template <int VEC, int LG>
static int launch_xent_stripes(cudaStream_t st, ane_idtype idtype, int B, int V, int S, float *dlogits, const float *logits,
                               const void *targets, float *loss_tok, float grad_scale, ane_cuda_status *status, int cl) {
    const int tps = (S + LG * VEC - 1) / (LG * VEC);
    const unsigned n = (unsigned)(B * tps);
#define ANE_XENT_CL(CLV)                                                                                                              \
    return idtype == ANE_ID_U16 ? launch_xent_cl<uint16_t, VEC, LG, CLV>(st, n, V, S, tps, dlogits, logits, targets, loss_tok, grad_scale, status) \
                                : launch_xent_cl<int32_t, VEC, LG, CLV>(st, n, V, S, tps, dlogits, logits, targets, loss_tok, grad_scale, status)
    if constexpr (VEC == 4) {
        if (cl == 8) { ANE_XENT_CL(8); }
        if (cl == 4) { ANE_XENT_CL(4); }
        if (cl == 2) { ANE_XENT_CL(2); }
    }
    ANE_XENT_CL(1);
#undef ANE_XENT_CL
}

extern "C" {

int ane_cuda_cross_entropy_dev(void *stream, ane_idtype idtype, int B, int V, int S, float *dlogits, const float *logits,
                               const void *targets, float *loss_seq, float grad_scale) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dlogits && logits && targets && loss_seq, "%s: null pointer", __func__);
    ANE_REQUIRE(idtype == ANE_ID_U16 || idtype == ANE_ID_I32, "%s: bad id type", __func__);
    ANE_REQUIRE(B >= 1 && V >= 1 && S >= 1, "%s: bad shape B=%d V=%d S=%d", __func__, B, V, S);
    ANE_REQUIRE((long long)B * S < 0x7fffffffLL, "%s: too many tokens", __func__);
    ANE_CHECK_EXTENT(dlogits, (size_t)B * V * S * 4); ANE_CHECK_EXTENT(logits, (size_t)B * V * S * 4);
    ANE_CHECK_EXTENT(targets, (size_t)B * S * (idtype == ANE_ID_U16 ? 2 : 4)); ANE_CHECK_EXTENT(loss_seq, (size_t)B * 4);
    cudaStream_t st = (cudaStream_t)stream;
    float *loss_tok = static_cast<float *>(workspace((size_t)B * S * sizeof(float)));
    if (!loss_tok) return fail(ANE_CUDA_ERR_NOMEM, "%s: no scratch", __func__);
    ane_cuda_status *status = ctx().status;
    const bool vec = (S % 4 == 0) && aligned16(dlogits) && aligned16(logits);
    if (vec && tuning("xent_cluster", 0) && V >= 4096 && S % XC_TW == 0) {
        // persistent clusters of 8 blocks per 16-token stripe, most of the stripe resident in shared memory.  In-place
        // use (dlogits == logits) is fine: a stripe is read, prefetched and written by one cluster only.
        const int threads = tuning("xent_threads", 1024) == 512 ? 512 : 1024;
        const int sps = S / XC_TW;
        const long long nstripes = (long long)B * sps;
        const int rows_per_cta = (V + XC_CL - 1) / XC_CL;
        const int cap = tuning("xent_boxes", threads == 512 ? 6 : 12);  // 16 KB units; 12 = 192 KB
        int rows_res = rows_per_cta;
        if (rows_res > cap * XC_UNIT) rows_res = cap * XC_UNIT;
        const size_t smem = (size_t)rows_res * XC_TW * sizeof(float) + 128;
        if (nstripes < 0x7fffffffLL && cap >= 0 && cap <= XC_MAXUNITS) {
            void (*kern)(float *, const float *, const void *, float *, int, int, int, int, int, int, float, ane_cuda_status *);
            if (threads == 512) kern = idtype == ANE_ID_U16 ? xent_cluster_kernel<uint16_t, 512> : xent_cluster_kernel<int32_t, 512>;
            else kern = idtype == ANE_ID_U16 ? xent_cluster_kernel<uint16_t, 1024> : xent_cluster_kernel<int32_t, 1024>;
            ANE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            // how many clusters can be resident at once
            cudaLaunchConfig_t cfgq = {};
            cfgq.gridDim = dim3(XC_CL * 64);
            cfgq.blockDim = dim3(threads);
            cfgq.dynamicSmemBytes = smem;
            cudaLaunchAttribute at;
            at.id = cudaLaunchAttributeClusterDimension;
            at.val.clusterDim.x = XC_CL; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
            cfgq.attrs = &at;
            cfgq.numAttrs = 1;
            int max_clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfgq) != cudaSuccess || max_clusters < 1) { cudaGetLastError(); max_clusters = 8; }
            int ncl = (long long)max_clusters < nstripes ? max_clusters : (int)nstripes;
            kern<<<(unsigned)(ncl * XC_CL), threads, smem, st>>>(dlogits, logits, targets, loss_tok, V, S, sps, (int)nstripes, rows_per_cta,
                                                                rows_res, grad_scale, status);
            xent_loss_kernel<<<B, 256, 0, st>>>(loss_seq, loss_tok, S);
            ANE_LAUNCH_OK(2);
            return ANE_CUDA_OK;
        }
    }
    // Stripes of 64 tokens (256-byte rows: measured 0.64 of the copy rate against 0.57 with 128-byte rows and 0.53 with
    // 64-byte rows); when that gives fewer than four blocks per SM, clusters of 2, 4 or 8 blocks share a stripe's vocabulary.
    const int lg_knob = tuning("xent_lg", S >= 64 ? 16 : 8);
    const int lg_eff = !vec ? 32 : (lg_knob == 4 || lg_knob == 16 || lg_knob == 32) ? lg_knob : 8;
    const long long nstripes_ = (long long)B * ((S + lg_eff * (vec ? 4 : 1) - 1) / (lg_eff * (vec ? 4 : 1)));
    int cl_auto = 1;
    while (cl_auto < 8 && nstripes_ * cl_auto < 4LL * ctx().sm_count && V / (2 * cl_auto) >= 2048) cl_auto *= 2;
    // A small vocabulary (a stripe of at most 4 MB): with eight blocks per stripe the rows held by the blocks that are
    // resident at one time come to about 150 MB instead of 1.2 GB, near the size of L2, and the reversed second sweep finds
    // a good part of its rows there: 0.676 of the copy rate against 0.647 for V = 9200.  Fewer resident blocks, to shrink
    // that set further, lose more bandwidth than the hits return (0.58 with three blocks per SM, 0.48 with two).
    if (vec && (long long)V * lg_eff * 16 <= (4LL << 20) && V >= 8 * 64) cl_auto = 8;
    const int cl = vec ? tuning("xent_split", cl_auto) : 1;
    int rc;
    if (!vec) rc = launch_xent_stripes<1, 32>(st, idtype, B, V, S, dlogits, logits, targets, loss_tok, grad_scale, status, 1);
    else if (lg_eff == 4) rc = launch_xent_stripes<4, 4>(st, idtype, B, V, S, dlogits, logits, targets, loss_tok, grad_scale, status, cl);
    else if (lg_eff == 16) rc = launch_xent_stripes<4, 16>(st, idtype, B, V, S, dlogits, logits, targets, loss_tok, grad_scale, status, cl);
    else if (lg_eff == 32) rc = launch_xent_stripes<4, 32>(st, idtype, B, V, S, dlogits, logits, targets, loss_tok, grad_scale, status, cl);
    else rc = launch_xent_stripes<4, 8>(st, idtype, B, V, S, dlogits, logits, targets, loss_tok, grad_scale, status, cl);
    if (rc != ANE_CUDA_OK) return rc;
    xent_loss_kernel<<<B, 256, 0, st>>>(loss_seq, loss_tok, S);
    ANE_LAUNCH_OK(2);
    return ANE_CUDA_OK;
}

}  // extern "C"
