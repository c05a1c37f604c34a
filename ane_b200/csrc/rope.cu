// rope.cu -- rotary position embedding (interleaved channel pairs), per-head QK-RMSNorm, and
// their fusions: qknorm -> rope (forward) and rope^-1 -> qknorm_bwd (backward).
//
// Tensors are [B][heads*hd][S].  A block owns a token tile of LG*VEC tokens of one sequence
// and walks over the heads; inside a head the THREADS/LG row groups each hold RPT consecutive
// channels (so both channels of a rotation pair sit in one thread) in registers between the
// per-token reduction and the write: every byte crosses HBM once.  sin/cos for the thread's
// pairs and tokens are computed once per tile and reused for every head.
#include "common.cuh"
#include "tma.cuh"

#include <math.h>
#include <type_traits>
#include <initializer_list>

namespace ane {

int rmsnorm_fwd_any(cudaStream_t st, ane_dtype dtype, int B, int C, int S, void *out, const void *x, const float *w, float eps);
int rmsnorm_bwd_any(cudaStream_t st, ane_dtype dtype, int B, int C, int S, void *dx, float *dw, const void *dy,
                    const void *x, const float *w, const void *add, float eps, unsigned flags);

constexpr int QK_THREADS = 256;
#ifndef ANE_QK_BWD_PIPE_DEFAULT
#define ANE_QK_BWD_PIPE_DEFAULT 1
#endif

// ------------------------------------------------------------------ cos / sin table
// theta(t, i) = (pos0 + t) * freq[i] depends on neither the head nor the sequence, but evaluating
// cosf / sinf per thread and tile costs as many instructions as all the rest of a fused kernel.
// The values are therefore computed once, by the same expressions, into a table
// cos[i][t], sin[i][t] (i < hd/2, t < S) that stays L2-resident, and cached per
// (hd, S, base, pos0) on the device.
__global__ void rope_table_kernel(float *__restrict__ cosT, float *__restrict__ sinT, int S, int half, int pos0,
                                  const __grid_constant__ RopeFreq freq) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= S * half) return;
    const int i = idx / S, t = idx % S;
    const float theta = (float)(pos0 + t) * freq.f[i];
    cosT[idx] = cosf(theta);
    sinT[idx] = sinf(theta);
}

// A table that was handed out is never freed, moved or refilled with other contents before ane_cuda_shutdown (or
// ane_cuda_release_caches): a kernel already enqueued or a CUDA graph already captured may hold its address.
struct RopeTable { int hd, S, pos0; float base; float *dev; cudaEvent_t filled; cudaStream_t filled_on; };
constexpr int ROPE_MAX_TABLES = 64;
static RopeTable g_tables[ROPE_MAX_TABLES] = {};
static int g_ntables = 0;

void rope_tables_release() {
    for (int i = 0; i < g_ntables; i++) {
        if (g_tables[i].dev) cudaFree(g_tables[i].dev);
        if (g_tables[i].filled) cudaEventDestroy(g_tables[i].filled);
        g_tables[i] = RopeTable();
    }
    g_ntables = 0;
}

// Returns the cos table (the sin table follows at + S*hd/2 floats), or nullptr with *rc set.
static const float *rope_table(cudaStream_t st, int hd, int S, float base, int pos0, const RopeFreq &fq, int *rc, const char *who) {
    for (int i = 0; i < g_ntables; i++) {
        RopeTable &t = g_tables[i];
        if (t.hd == hd && t.S == S && t.pos0 == pos0 && t.base == base) {
            // filled on another stream: order this stream after the fill unless it is known to be complete.  Not while
            // this stream is being captured: a table used in a capture was filled by an eager call before it, and the
            // capture's own start already comes after the caller's synchronisation with that call.
            if (t.filled_on != st) {
                cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
                if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) cudaGetLastError();
                if (cap == cudaStreamCaptureStatusNone && cudaEventQuery(t.filled) != cudaSuccess) {
                    cudaGetLastError();
                    cudaStreamWaitEvent(st, t.filled, 0);
                }
            }
            return t.dev;
        }
    }
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) cudaGetLastError();
    if (cap != cudaStreamCaptureStatusNone) {
        *rc = fail(ANE_CUDA_ERR_UNSUPPORTED, "%s: no cos/sin table for (head width %d, S %d, base %g, first position %d) yet and the stream is "
                   "being captured; run the operator once with these arguments before capturing", who, hd, S, (double)base, pos0);
        return nullptr;
    }
    if (frozen()) {
        *rc = fail(ANE_CUDA_ERR_UNSUPPORTED, "%s: no cos/sin table for (head width %d, S %d, base %g, first position %d) and the library is "
                   "frozen (ane_cuda_freeze)", who, hd, S, (double)base, pos0);
        return nullptr;
    }
    if (g_ntables == ROPE_MAX_TABLES) {
        *rc = fail(ANE_CUDA_ERR_UNSUPPORTED, "%s: %d distinct cos/sin tables are cached; call ane_cuda_release_caches() once no enqueued work "
                   "or captured graph uses them", who, ROPE_MAX_TABLES);
        return nullptr;
    }
    RopeTable &t = g_tables[g_ntables];
    const size_t n = (size_t)S * (hd / 2);
    float *dev = nullptr;
    if (dev_malloc(reinterpret_cast<void **>(&dev), 2 * n * sizeof(float)) != cudaSuccess) {
        *rc = fail(ANE_CUDA_ERR_NOMEM, "%s: no memory for the cos/sin table", who);
        return nullptr;
    }
    cudaEvent_t ev = nullptr;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(dev);
        *rc = fail(ANE_CUDA_ERR_CUDA, "%s: cudaEventCreate failed", who);
        return nullptr;
    }
    rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(dev, dev + n, S, hd / 2, pos0, fq);
    cudaEventRecord(ev, st);
    note_launch(1);
    t = RopeTable{hd, S, pos0, base, dev, ev, st};
    g_ntables++;
    return dev;
}

// ------------------------------------------------------------------ stand-alone RoPE
// One thread: one pair index i, VEC tokens, all heads.   cpu_ops.h:168-184 / forward.h:55-70
// cos / sin come from the cached table when there is one (cosT != nullptr; vector path only), else from the same
// cosf / sinf expressions evaluated here -- the same bits either way.
template <int N> __device__ __forceinline__ V<N> table_lanes(const float *p);
template <typename T, int VEC, int LG>
__global__ void __launch_bounds__(QK_THREADS)
rope_kernel(T *out, const T *x, int heads, int hd, int S, int tiles_per_seq, int pos0, bool inverse,
            const __grid_constant__ RopeFreq freq, const float *__restrict__ cosT, const float *__restrict__ sinT) {
    constexpr int R = QK_THREADS / LG;
    constexpr int TW = LG * VEC;
    const int b = blockIdx.x / tiles_per_seq;
    const int lg = threadIdx.x % LG, rg = threadIdx.x / LG;
    const int t = (blockIdx.x % tiles_per_seq) * TW + lg * VEC;
    if (t >= S) return;
    const int C = heads * hd;
    const size_t base = (size_t)b * C * S + t;
    const size_t hstep = (size_t)hd * S;
    for (int i = blockIdx.y * R + rg; i < hd / 2; i += gridDim.y * R) {
        V<VEC> cs, sn;
        bool from_table = false;
        if constexpr (VEC >= 4) {
            if (cosT) {
                cs = table_lanes<VEC>(cosT + (size_t)i * S + t);
                sn = table_lanes<VEC>(sinT + (size_t)i * S + t);
                if (inverse) {
#pragma unroll
                    for (int q = 0; q < VEC / 2; q++) sn.p[q] = make_float2(-sn.p[q].x, -sn.p[q].y);
                }
                from_table = true;
            }
        }
        if (!from_table) {
            const float fr = freq.f[i];
#pragma unroll
            for (int j = 0; j < VEC; j++) {
                const float theta = (float)(pos0 + t + j) * fr;
                cs.set(j, cosf(theta));
                sn.set(j, inverse ? -sinf(theta) : sinf(theta));
            }
        }
        const size_t o0 = base + (size_t)(2 * i) * S;
        int h = 0;
        for (; h + 2 <= heads; h += 2) {          // two heads (four rows) in flight
            Raw<T, VEC> r0, r1, r2, r3;
            const size_t o = o0 + h * hstep;
            r0.load_stream(x + o);
            r1.load_stream(x + o + S);
            r2.load_stream(x + o + hstep);
            r3.load_stream(x + o + hstep + S);
            const V<VEC> a0 = r0.get(), b0 = r1.get(), a1 = r2.get(), b1 = r3.get();
            r0.put(vsub(vmul(a0, cs), vmul(b0, sn)));
            r1.put(vfma(a0, sn, vmul(b0, cs)));
            r2.put(vsub(vmul(a1, cs), vmul(b1, sn)));
            r3.put(vfma(a1, sn, vmul(b1, cs)));
            r0.store_stream(out + o);
            r1.store_stream(out + o + S);
            r2.store_stream(out + o + hstep);
            r3.store_stream(out + o + hstep + S);
        }
        for (; h < heads; h++) {
            Raw<T, VEC> r0, r1;
            const size_t o = o0 + h * hstep;
            r0.load_stream(x + o);
            r1.load_stream(x + o + S);
            const V<VEC> a0 = r0.get(), b0 = r1.get();
            r0.put(vsub(vmul(a0, cs), vmul(b0, sn)));
            r1.put(vfma(a0, sn, vmul(b0, cs)));
            r0.store_stream(out + o);
            r1.store_stream(out + o + S);
        }
    }
}

// ------------------------------------------------------------------ fused per-head kernels
// hd == RPT * 32; a block of 256 threads owns a tile of 8*VEC tokens and walks over the heads,
// HB heads per step.  Thread (rg, lg) holds channels rg*RPT .. rg*RPT+RPT-1 of each head of the
// step (both channels of a rotation pair sit in one thread) for its VEC tokens, in registers,
// from the load to the store.  sin/cos for the thread's pairs and tokens are computed once per
// tile and reused for every head.
// N consecutive table entries (16-byte aligned) as packed lanes.
template <int N> __device__ __forceinline__ V<N> table_lanes(const float *p) {
    V<N> v;
#pragma unroll
    for (int i = 0; i < N / 4; i++) {
        const float4 q = __ldg(reinterpret_cast<const float4 *>(p) + i);
        v.p[2 * i] = make_float2(q.x, q.y);
        v.p[2 * i + 1] = make_float2(q.z, q.w);
    }
    return v;
}

constexpr int QK_LG = 8;
constexpr int QK_R = QK_THREADS / QK_LG;   // 32 row groups

template <typename T, int RPT, bool ROPE, int HB>
__global__ void __launch_bounds__(QK_THREADS, 2)
qk_fwd_kernel(T *__restrict__ out, const T *__restrict__ x, const float *__restrict__ w, int heads, int S,
              int tiles_per_seq, float eps, const float *__restrict__ cosT, const float *__restrict__ sinT) {
    constexpr int VEC = Elt<T>::VEC;
    constexpr int TW = QK_LG * VEC;
    constexpr int HD = RPT * QK_R;
    __shared__ __align__(16) float red[2][HB][QK_R][TW];
    __shared__ __align__(16) float tot[2][HB][TW];

    const int b = blockIdx.x / tiles_per_seq;
    const int lg = threadIdx.x % QK_LG, rg = threadIdx.x / QK_LG;
    const int t = (blockIdx.x % tiles_per_seq) * TW + lg * VEC;
    const bool active = t < S;
    const size_t base = (size_t)b * heads * HD * S + t + (size_t)(rg * RPT) * S;
    const size_t hstep = (size_t)HD * S;
    const float invd = 1.0f / (float)HD;

    float wc[RPT];
#pragma unroll
    for (int k = 0; k < RPT; k++) wc[k] = __ldg(w + rg * RPT + k);

    V<VEC> cs[RPT / 2], sn[RPT / 2];
    if (ROPE && active) {
#pragma unroll
        for (int p = 0; p < RPT / 2; p++) {
            cs[p] = table_lanes<VEC>(cosT + (size_t)(rg * (RPT / 2) + p) * S + t);
            sn[p] = table_lanes<VEC>(sinT + (size_t)(rg * (RPT / 2) + p) * S + t);
        }
    }

    int it = 0;
    for (int h0 = 0; h0 < heads; h0 += HB, it++) {
        const int buf = it & 1;
        Raw<T, VEC> r[HB][RPT];
#pragma unroll
        for (int hh = 0; hh < HB; hh++)
            if (active && h0 + hh < heads) {
#pragma unroll
                for (int k = 0; k < RPT; k++) r[hh][k].load_stream(x + base + (h0 + hh) * hstep + (size_t)k * S);
            }
#pragma unroll
        for (int hh = 0; hh < HB; hh++) {
            V<VEC> ss = V<VEC>::splat(0.0f);
            if (active && h0 + hh < heads) {
#pragma unroll
                for (int k = 0; k < RPT; k++) { const V<VEC> v = r[hh][k].get(); ss = vfma(v, v, ss); }
            }
            lanes_to_smem<VEC>(&red[buf][hh][rg][lg * VEC], ss);
        }
        __syncthreads();
#pragma unroll
        for (int hh = 0; hh < HB; hh++) {     // column sums with the whole block, then rrms once per token
            constexpr int P = QK_THREADS / TW;
            const float s = block_column_sum<QK_R, TW, QK_THREADS>(&red[buf][hh][0][0], threadIdx.x);
            if (threadIdx.x % P == 0) tot[buf][hh][threadIdx.x / P] = 1.0f / sqrtf(__fadd_rn(__fmul_rn(s, invd), eps));
        }
        __syncthreads();
#pragma unroll
        for (int hh = 0; hh < HB; hh++) {
            if (active && h0 + hh < heads) {
                const V<VEC> rr = lanes_from_smem<VEC>(&tot[buf][hh][lg * VEC]);
                V<VEC> v[RPT];
#pragma unroll
                for (int k = 0; k < RPT; k++) v[k] = vscale(vmul(r[hh][k].get(), rr), wc[k]);
                if (ROPE) {
#pragma unroll
                    for (int p = 0; p < RPT / 2; p++) {
                        const V<VEC> a = v[2 * p], bb = v[2 * p + 1];
                        v[2 * p] = vsub(vmul(a, cs[p]), vmul(bb, sn[p]));
                        v[2 * p + 1] = vfma(a, sn[p], vmul(bb, cs[p]));
                    }
                }
#pragma unroll
                for (int k = 0; k < RPT; k++) {
                    Raw<T, VEC> o;
                    o.put(v[k]);
                    o.store_stream(out + base + (h0 + hh) * hstep + (size_t)k * S);
                }
            }
        }
    }
}

template <typename T, int RPT, bool ROPE, int HB>
__global__ void __launch_bounds__(QK_THREADS, (HB == 1 ? 2 : 1))
qk_bwd_kernel(T *__restrict__ dx, float *__restrict__ partial, const T *__restrict__ dy, const T *__restrict__ x,
              const float *__restrict__ w, int heads, int S, int tiles_per_seq, int ntiles, float eps,
              unsigned flags, const float *__restrict__ cosT, const float *__restrict__ sinT) {
    constexpr int VEC = Elt<T>::VEC;
    constexpr int TW = QK_LG * VEC;
    constexpr int HD = RPT * QK_R;
    __shared__ __align__(16) float red[2][HB][2][QK_R][TW];
    __shared__ __align__(16) float tot[2][HB][2][TW];

    const int lg = threadIdx.x % QK_LG, rg = threadIdx.x / QK_LG;
    const float invd = 1.0f / (float)HD;
    const bool exact = (flags & ANE_NORM_BWD_EXACT) != 0;
    const size_t hstep = (size_t)HD * S;

    float wc[RPT], dwacc[RPT];
#pragma unroll
    for (int k = 0; k < RPT; k++) { wc[k] = __ldg(w + rg * RPT + k); dwacc[k] = 0.0f; }

    int it = 0;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int b = tile / tiles_per_seq;
        const int t = (tile % tiles_per_seq) * TW + lg * VEC;
        const bool active = t < S;
        const size_t base = (size_t)b * heads * HD * S + t + (size_t)(rg * RPT) * S;

        V<VEC> cs[RPT / 2], sn[RPT / 2];
        if (ROPE && active) {
#pragma unroll
            for (int p = 0; p < RPT / 2; p++) {
                cs[p] = table_lanes<VEC>(cosT + (size_t)(rg * (RPT / 2) + p) * S + t);
                sn[p] = table_lanes<VEC>(sinT + (size_t)(rg * (RPT / 2) + p) * S + t);
            }
        }

        for (int h0 = 0; h0 < heads; h0 += HB, it++) {
            const int buf = it & 1;
            Raw<T, VEC> rxr[HB][RPT], rdr[HB][RPT];
#pragma unroll
            for (int hh = 0; hh < HB; hh++)
                if (active && h0 + hh < heads) {
#pragma unroll
                    for (int k = 0; k < RPT; k++) {
                        rxr[hh][k].load_stream(x + base + (h0 + hh) * hstep + (size_t)k * S);
                        rdr[hh][k].load_stream(dy + base + (h0 + hh) * hstep + (size_t)k * S);
                    }
                }
            // g = rope^-1(dy): (a cos + b sin, -a sin + b cos)   cpu_ops.h:178-181 ; kept packed in rdr
#pragma unroll
            for (int hh = 0; hh < HB; hh++) {
                V<VEC> ss = V<VEC>::splat(0.0f), dot = V<VEC>::splat(0.0f);
                if (active && h0 + hh < heads) {
#pragma unroll
                    for (int p = 0; p < RPT / 2; p++) {
                        V<VEC> g0 = rdr[hh][2 * p].get(), g1 = rdr[hh][2 * p + 1].get();
                        if (ROPE) {
                            const V<VEC> a = g0, bb = g1;
                            g0 = vfma(a, cs[p], vmul(bb, sn[p]));
                            g1 = vsub(vmul(bb, cs[p]), vmul(a, sn[p]));
                        }
                        const V<VEC> x0 = rxr[hh][2 * p].get(), x1 = rxr[hh][2 * p + 1].get();
                        ss = vfma(x0, x0, ss);
                        ss = vfma(x1, x1, ss);
                        dot = vfma_s(vmul(g0, x0), wc[2 * p], dot);
                        dot = vfma_s(vmul(g1, x1), wc[2 * p + 1], dot);
                    }
                }
                lanes_to_smem<VEC>(&red[buf][hh][0][rg][lg * VEC], ss);
                lanes_to_smem<VEC>(&red[buf][hh][1][rg][lg * VEC], dot);
            }
            __syncthreads();
#pragma unroll
            for (int hh = 0; hh < HB; hh++) {  // column sums with the whole block, then rrms and coef once per token
                constexpr int P = QK_THREADS / TW;
                const float s0 = block_column_sum<QK_R, TW, QK_THREADS>(&red[buf][hh][0][0][0], threadIdx.x);
                const float s1 = block_column_sum<QK_R, TW, QK_THREADS>(&red[buf][hh][1][0][0], threadIdx.x);
                if (threadIdx.x % P == 0) {
                    const float r1 = 1.0f / sqrtf(__fadd_rn(__fmul_rn(s0, invd), eps));
                    float r2 = r1 * r1;
                    r2 = r2 * invd;
                    tot[buf][hh][0][threadIdx.x / P] = r1;
                    tot[buf][hh][1][threadIdx.x / P] = s1 * r2;
                }
            }
            __syncthreads();
#pragma unroll
            for (int hh = 0; hh < HB; hh++) {
                if (active && h0 + hh < heads) {
                    const V<VEC> rr = lanes_from_smem<VEC>(&tot[buf][hh][0][lg * VEC]);
                    const V<VEC> coef = lanes_from_smem<VEC>(&tot[buf][hh][1][lg * VEC]);
#pragma unroll
                    for (int p = 0; p < RPT / 2; p++) {
                        V<VEC> g[2];
                        g[0] = rdr[hh][2 * p].get();
                        g[1] = rdr[hh][2 * p + 1].get();
                        if (ROPE) {     // recomputed rather than kept: registers are the scarcer resource
                            const V<VEC> a = g[0], bb = g[1];
                            g[0] = vfma(a, cs[p], vmul(bb, sn[p]));
                            g[1] = vsub(vmul(bb, cs[p]), vmul(a, sn[p]));
                        }
#pragma unroll
                        for (int q = 0; q < 2; q++) {
                            const int k = 2 * p + q;
                            const V<VEC> xv = rxr[hh][k].get();
                            V<VEC> o;
                            if (exact) o = vmul(vsub(vscale(g[q], wc[k]), vmul(xv, coef)), rr);
                            else o = vscale(vmul(vsub(g[q], vmul(xv, coef)), rr), wc[k]);
                            dwacc[k] += vmul(vmul(g[q], xv), rr).hsum();
                            Raw<T, VEC> ro;
                            ro.put(o);
                            ro.store_stream(dx + base + (h0 + hh) * hstep + (size_t)k * S);
                        }
                    }
                }
            }
        }
    }
    // dw partial of this block: sum the LG lanes of each row group, fixed order
#pragma unroll
    for (int k = 0; k < RPT; k++) {
        float s = dwacc[k];
#pragma unroll
        for (int off = QK_LG / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (lg == 0) partial[(size_t)blockIdx.x * HD + rg * RPT + k] = s;
    }
}

// ------------------------------------------------------------------ TMA-fed variants
// Same thread layout and arithmetic as qk_fwd_kernel / qk_bwd_kernel, but the head tiles
// ([HD channels x 8*VEC tokens], 16 KiB in bf16) are brought into a ring of NST shared-memory
// stages by the tensor copy engine, several tiles ahead of the math: loads stay in flight all the
// time and cost no registers.  A block is persistent over token tiles; within a tile it walks
// over the heads.  Thread 0 issues the copies; a stage is refilled right after the block-wide
// barrier that follows everybody's read of it (the barrier the reduction needs anyway).
// Waits on the copy barriers are bounded: on a give-up the block records it in the status words
// and returns.
struct ItemMap {
    int heads, grid, bid, n_full, lo, n_items, first_left_tile;
    __device__ ItemMap(int ntiles, int heads_, int grid_, int bid_) : heads(heads_), grid(grid_), bid(bid_) {
        const int rounds = ntiles / grid;
        n_full = rounds * heads;
        first_left_tile = rounds * grid;
        const int left = (ntiles - first_left_tile) * heads;            // items of the partial round
        const int per = (left + grid - 1) / grid;
        lo = bid * per;
        int hi = lo + per < left ? lo + per : left;
        n_items = n_full + (hi > lo ? hi - lo : 0);
    }
    // (tile, head) of item 0, then of item j_next given those of item j_next - 1: no division per item
    __device__ __forceinline__ void first(int &tl, int &h) const {
        if (n_full > 0) { tl = bid; h = 0; }
        else { tl = first_left_tile + lo / heads; h = lo % heads; }
    }
    __device__ __forceinline__ void next(int j_next, int &tl, int &h) const {
        if (j_next == n_full) { tl = first_left_tile + lo / heads; h = lo % heads; return; }
        if (++h == heads) { h = 0; tl += j_next < n_full ? grid : 1; }
    }
};

template <typename T, int RPT, bool ROPE, int NST, bool TILED = false, bool PIPE = true>
__global__ void __launch_bounds__(QK_THREADS)
qk_fwd_tma_kernel(T *__restrict__ out, const __grid_constant__ CUtensorMap xmap, const float *__restrict__ w, int heads,
                  int S, int tiles_per_seq, int ntiles, float eps, ane_cuda_status *status,
                  const float *__restrict__ cosT, const float *__restrict__ sinT, int out_ratio, RingTest test) {
    constexpr int VEC = Elt<T>::VEC;
    constexpr int TW = QK_LG * VEC;
    constexpr int HD = RPT * QK_R;
    constexpr uint32_t STAGE_BYTES = HD * TW * sizeof(T);
    extern __shared__ unsigned char stages_raw[];
    unsigned char *stages = stages_raw + ((128u - (smem_u32(stages_raw) & 127u)) & 127u);   // 128-byte aligned copy targets
    __shared__ __align__(8) uint64_t full[NST];
    __shared__ __align__(16) float red[2][QK_R][TW];
    __shared__ __align__(16) float tot[2][TW];
    __shared__ int give_up;

    const int lg = threadIdx.x % QK_LG, rg = threadIdx.x / QK_LG;
    const float invd = 1.0f / (float)HD;
    const size_t hstep = (size_t)HD * S;
    // Work items are (token tile, head) pairs.  Full rounds: block i takes tile r*grid + i with all its
    // heads, so the blocks running at one time sit on neighbouring token tiles of the same rows (DRAM page
    // locality).  The tiles left after the last full round are shared out head by head, so no block idles
    // for a whole tile.
    const ItemMap im(ntiles, heads, (int)gridDim.x, (int)blockIdx.x);
    const int n_items = im.n_items;

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < NST; s++) mbar_init(&full[s], 1);
        mbar_init_fence();
        give_up = 0;
    }
    __syncthreads();
    dep_sync();                          // nothing above touches global memory

    int ptl, ph, ctl, ch;                // producer (thread 0) and consumer positions
    im.first(ctl, ch);
    im.first(ptl, ph);
    int issued = 0;                      // thread 0: items whose copies have been started
    auto issue = [&](int j) {
        const int tl = ptl;
        const int s = j % NST;
        mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
        if (j != test.skip_item)
            tma_load_3d(stages + (size_t)s * STAGE_BYTES, &xmap, (tl % tiles_per_seq) * TW, ph * HD, tl / tiles_per_seq, &full[s]);
        im.next(j + 1, ptl, ph);
        issued = j + 1;
    };
    // After a give-up nothing may still be in flight into this block's shared memory when it exits: thread 0 waits
    // (bounded) for every later item whose copy was started.
    auto drain = [&](int j) {
        for (int jj = j + 1; jj < issued; jj++)
            if (jj != test.skip_item) mbar_wait_bounded(&full[jj % NST], (uint32_t)(jj / NST) & 1u, test.wait_limit);
    };
    if (threadIdx.x == 0)
        for (int j = 0; j < NST && j < n_items; j++) issue(j);

    float wc[RPT];
#pragma unroll
    for (int k = 0; k < RPT; k++) wc[k] = __ldg(w + rg * RPT + k);
    V<VEC> cs[RPT / 2], sn[RPT / 2];

    // Scale, rotate and store the rows `r` of an item whose reciprocal norms are in tot[buf].
    auto finish_item = [&](const Raw<T, VEC> (&r)[RPT], int b, int h, int t, int buf) {
        const V<VEC> rr = lanes_from_smem<VEC>(&tot[buf][lg * VEC]);
        V<VEC> v[RPT];
#pragma unroll
        for (int k = 0; k < RPT; k++) v[k] = vscale(vmul(r[k].get(), rr), wc[k]);
        if (ROPE) {
#pragma unroll
            for (int p = 0; p < RPT / 2; p++) {
                const V<VEC> a = v[2 * p], bb = v[2 * p + 1];
                v[2 * p] = vsub(vmul(a, cs[p]), vmul(bb, sn[p]));
                v[2 * p + 1] = vfma(a, sn[p], vmul(bb, cs[p]));
            }
        }
        // out_ratio > 1: the result is written to the `out_ratio` query heads that share this KV head (the tiled
        // layout of a grouped-query model, training_dynamic/io.h:330-337, as an index map instead of a copy)
        const int n_out = TILED ? out_ratio : 1;
        for (int q = 0; q < n_out; q++) {
            const size_t o = TILED ? ((size_t)b * heads * out_ratio + (size_t)h * out_ratio + q) * hstep + (size_t)(rg * RPT) * S + t
                                   : (size_t)b * heads * hstep + h * hstep + (size_t)(rg * RPT) * S + t;
#pragma unroll
            for (int k = 0; k < RPT; k++) {
                Raw<T, VEC> ro;
                ro.put(v[k]);
                ro.store_stream(out + o + (size_t)k * S);
            }
        }
    };
    auto load_table = [&](int t) {
#pragma unroll
        for (int p = 0; p < RPT / 2; p++) {
            cs[p] = table_lanes<VEC>(cosT + (size_t)(rg * (RPT / 2) + p) * S + t);
            sn[p] = table_lanes<VEC>(sinT + (size_t)(rg * (RPT / 2) + p) * S + t);
        }
    };

    // PIPE: one block barrier per item instead of two.  Iteration j reads item j from its stage and publishes its partial
    // sums; after the barrier the reciprocal norms of item j are made, and item j-1 -- whose rows are still in registers and
    // whose norms were made one barrier ago -- is scaled, rotated and stored.  The loads and sums of one item thus overlap the
    // arithmetic and stores of the one before it.  red / tot alternate between two buffers, which the single barrier per
    // item keeps apart (a buffer is rewritten two barriers after it was last read).
    Raw<T, VEC> rp[RPT];
    int pb = 0, phd = 0, pt = 0, pbuf = 0;
    bool pactive = false;

    int b = 0, t = 0;                    // sequence and first token of the current tile: one division per tile, not per item
    bool active = false;
    for (int j = 0; j < n_items; j++) {
        const int tl = ctl, h = ch;
        im.next(j + 1, ctl, ch);
        const int s = j % NST, buf = j & 1;
        const bool new_tile = h == 0 || j == 0 || j == im.n_full;
        if (new_tile) {
            b = tl / tiles_per_seq;
            t = (tl - b * tiles_per_seq) * TW + lg * VEC;
            active = t < S;
        }
        if (!PIPE && ROPE && new_tile && active) load_table(t);
        if (!mbar_wait_bounded(&full[s], (uint32_t)(j / NST) & 1u, test.wait_limit)) atomicExch(&give_up, 1);
        const T *tile = reinterpret_cast<const T *>(stages + (size_t)s * STAGE_BYTES);
        Raw<T, VEC> r[RPT];
        V<VEC> ss = V<VEC>::splat(0.0f);
#pragma unroll
        for (int k = 0; k < RPT; k++) {
            r[k].load(tile + (rg * RPT + k) * TW + lg * VEC);
            const V<VEC> v = r[k].get();
            ss = vfma(v, v, ss);
        }
        lanes_to_smem<VEC>(&red[buf][rg][lg * VEC], ss);
        __syncthreads();                                   // every thread has its part of stage s in registers
        if (*(volatile int *)&give_up) {
            if (threadIdx.x == 0) { atomicAdd(&status->wait_giveups, 1); drain(j); }
            return;
        }
        if (threadIdx.x == 0 && j + NST < n_items) { fence_proxy_async(); issue(j + NST); }
        {
            constexpr int P = QK_THREADS / TW;
            const float sum = block_column_sum<QK_R, TW, QK_THREADS>(&red[buf][0][0], threadIdx.x);
            if (threadIdx.x % P == 0) tot[buf][threadIdx.x / P] = 1.0f / sqrtf(__fadd_rn(__fmul_rn(sum, invd), eps));
        }
        if (PIPE) {
            if (j > 0 && pactive) finish_item(rp, pb, phd, pt, pbuf);
            if (ROPE && new_tile && active) load_table(t);       // the table of item j's tile: used one iteration later
#pragma unroll
            for (int k = 0; k < RPT; k++) rp[k] = r[k];
            pb = b; phd = h; pt = t; pbuf = buf; pactive = active;
        } else {
            __syncthreads();
            if (active) finish_item(r, b, h, t, buf);
        }
    }
    if (PIPE && n_items > 0) {
        __syncthreads();                                   // the norms of the last item
        if (pactive) finish_item(rp, pb, phd, pt, pbuf);
    }
}

// GQ > 1: dy is the TILED gradient [B][heads*GQ*HD][S] of a grouped-query layout (query head h*GQ + r belongs to
// KV head h); the GQ tiles of a head are added in fp32, in head order, and rounded once to T before anything else
// uses them -- exactly what gqa_reduce followed by this operator computes (training_dynamic/io.h:340-351,
// train.m:653-656), without the reduced tensor ever crossing HBM.
template <typename T, int RPT, bool ROPE, int NST, int GQ = 1, bool PIPE = false>
__global__ void __launch_bounds__(QK_THREADS, 2)
qk_bwd_tma_kernel(T *__restrict__ dx, float *__restrict__ partial, const __grid_constant__ CUtensorMap dymap,
                  const __grid_constant__ CUtensorMap xmap, const float *__restrict__ w, int heads, int S, int tiles_per_seq,
                  int ntiles, float eps, unsigned flags, ane_cuda_status *status,
                  const float *__restrict__ cosT, const float *__restrict__ sinT, RingTest test) {
    constexpr int VEC = Elt<T>::VEC;
    constexpr int TW = QK_LG * VEC;
    constexpr int HD = RPT * QK_R;
    constexpr uint32_t TILE_BYTES = HD * TW * sizeof(T);
    constexpr uint32_t STAGE_BYTES = (1 + GQ) * TILE_BYTES;   // x tile, then the dy tile(s)
    extern __shared__ unsigned char stages_raw[];
    unsigned char *stages = stages_raw + ((128u - (smem_u32(stages_raw) & 127u)) & 127u);   // 128-byte aligned copy targets
    __shared__ __align__(8) uint64_t full[NST];
    constexpr int NWARP = QK_THREADS / 32;
    __shared__ __align__(16) float red[2][2][NWARP][TW];       // per-warp sums (row groups of a warp are added by shuffles)
    __shared__ __align__(16) float tot[2][2][TW];
    __shared__ int give_up;

    const int lg = threadIdx.x % QK_LG, rg = threadIdx.x / QK_LG;
    const float invd = 1.0f / (float)HD;
    const bool exact = (flags & ANE_NORM_BWD_EXACT) != 0;
    const size_t hstep = (size_t)HD * S;
    // Work items are (token tile, head) pairs.  Full rounds: block i takes tile r*grid + i with all its
    // heads, so the blocks running at one time sit on neighbouring token tiles of the same rows (DRAM page
    // locality).  The tiles left after the last full round are shared out head by head, so no block idles
    // for a whole tile.
    const ItemMap im(ntiles, heads, (int)gridDim.x, (int)blockIdx.x);
    const int n_items = im.n_items;

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < NST; s++) mbar_init(&full[s], 1);
        mbar_init_fence();
        give_up = 0;
    }
    __syncthreads();
    dep_sync();                          // nothing above touches global memory

    int ptl, ph, ctl, ch;                // producer (thread 0) and consumer positions
    im.first(ctl, ch);
    im.first(ptl, ph);
    int issued = 0;                      // thread 0: items whose copies have been started
    auto issue = [&](int j) {
        const int tl = ptl;
        const int s = j % NST;
        unsigned char *dst = stages + (size_t)s * STAGE_BYTES;
        mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
        if (j != test.skip_item) {
            tma_load_3d(dst, &xmap, (tl % tiles_per_seq) * TW, ph * HD, tl / tiles_per_seq, &full[s]);
#pragma unroll
            for (int r = 0; r < GQ; r++)
                tma_load_3d(dst + (1 + r) * TILE_BYTES, &dymap, (tl % tiles_per_seq) * TW, (ph * GQ + r) * HD, tl / tiles_per_seq, &full[s]);
        }
        im.next(j + 1, ptl, ph);
        issued = j + 1;
    };
    // After a give-up nothing may still be in flight into this block's shared memory when it exits: thread 0 waits
    // (bounded) for every later item whose copies were started.
    auto drain = [&](int j) {
        for (int jj = j + 1; jj < issued; jj++)
            if (jj != test.skip_item) mbar_wait_bounded(&full[jj % NST], (uint32_t)(jj / NST) & 1u, test.wait_limit);
    };
    if (threadIdx.x == 0)
        for (int j = 0; j < NST && j < n_items; j++) issue(j);

    float wc[RPT], dwacc[RPT];
#pragma unroll
    for (int k = 0; k < RPT; k++) { wc[k] = __ldg(w + rg * RPT + k); dwacc[k] = 0.0f; }
    V<VEC> cs[RPT / 2], sn[RPT / 2];

    // x and (summed) dy rows of pair p of a staged item, dy already rotated back
    auto load_pair = [&](const T *xt, const T *dt, int p, V<VEC> &x0, V<VEC> &x1, V<VEC> &g0, V<VEC> &g1) {
        Raw<T, VEC> a0, a1, c0, c1;
        a0.load(xt + (rg * RPT + 2 * p) * TW + lg * VEC);
        a1.load(xt + (rg * RPT + 2 * p + 1) * TW + lg * VEC);
        c0.load(dt + (rg * RPT + 2 * p) * TW + lg * VEC);
        c1.load(dt + (rg * RPT + 2 * p + 1) * TW + lg * VEC);
        x0 = a0.get();
        x1 = a1.get();
        g0 = c0.get();
        g1 = c1.get();
        if (ROPE) {       // g = rope^-1(dy): (a cos + b sin, -a sin + b cos)   cpu_ops.h:178-181
            const V<VEC> a = g0, bb = g1;
            g0 = vfma(a, cs[p], vmul(bb, sn[p]));
            g1 = vsub(vmul(bb, cs[p]), vmul(a, sn[p]));
        }
    };
    // Sweep 2 of the item staged in stage `s`, whose (rrms, coef) are in tot[buf]: dx and the dw partial sums.  It reads the
    // tile again from shared memory and redoes the inverse rotation (a few packed operations) -- sweep 1 keeps nothing but
    // the two sums, and the register file then allows two blocks per SM.
    auto sweep2 = [&](int s, int buf, int b, int h, int t) {
        const T *xt = reinterpret_cast<const T *>(stages + (size_t)s * STAGE_BYTES);
        const T *dt = reinterpret_cast<const T *>(stages + (size_t)s * STAGE_BYTES + TILE_BYTES);
        const V<VEC> rr = lanes_from_smem<VEC>(&tot[buf][0][lg * VEC]);
        const V<VEC> coef = lanes_from_smem<VEC>(&tot[buf][1][lg * VEC]);
        const size_t o = (size_t)b * heads * hstep + h * hstep + (size_t)(rg * RPT) * S + t;
#pragma unroll
        for (int p = 0; p < RPT / 2; p++) {
            V<VEC> xv[2], g[2];
            load_pair(xt, dt, p, xv[0], xv[1], g[0], g[1]);
#pragma unroll
            for (int q = 0; q < 2; q++) {
                const int k = 2 * p + q;
                V<VEC> ov;
                if (exact) ov = vmul(vsub(vscale(g[q], wc[k]), vmul(xv[q], coef)), rr);
                else ov = vscale(vmul(vsub(g[q], vmul(xv[q], coef)), rr), wc[k]);
                dwacc[k] += vmul(vmul(g[q], xv[q]), rr).hsum();
                Raw<T, VEC> ro;
                ro.put(ov);
                ro.store_stream(dx + o + (size_t)k * S);
            }
        }
    };
    auto load_table = [&](int t) {
#pragma unroll
        for (int p = 0; p < RPT / 2; p++) {
            cs[p] = table_lanes<VEC>(cosT + (size_t)(rg * (RPT / 2) + p) * S + t);
            sn[p] = table_lanes<VEC>(sinT + (size_t)(rg * (RPT / 2) + p) * S + t);
        }
    };

    // PIPE: sweep 2 of item j-1 runs AFTER sweep 1 of item j, behind the same barrier, so an item costs one block barrier
    // instead of two and the loads and sums of one item overlap the arithmetic and stores of the one before it.  Both sweeps
    // use the cos / sin values of their token tile, which live in registers once: where item j opens a new token tile, item
    // j-1 is finished first (one extra barrier per tile).  A stage is refilled one barrier after its item's sweep 2.
    int pend_s = 0, pend_buf = 0, pend_b = 0, pend_h = 0, pend_t = 0;     // item whose sweep 2 is still to run
    bool pend = false, pend_active = false;
    int freed = -1;                      // thread 0: every item <= freed has had its sweep 2 run by all threads (as of the last barrier)
    int next_issue = n_items < NST ? n_items : NST;

    int b = 0, t = 0;                    // sequence and first token of the current tile: one division per tile, not per item
    bool active = false;
    for (int j = 0; j < n_items; j++) {
        const int tl = ctl, h = ch;
        im.next(j + 1, ctl, ch);
        const int s = j % NST, buf = j & 1;
        const bool new_tile = h == 0 || j == 0 || j == im.n_full;
        if (new_tile) {
            b = tl / tiles_per_seq;
            t = (tl - b * tiles_per_seq) * TW + lg * VEC;
            active = t < S;
        }
        bool flushed = false;
        if (PIPE && pend && ROPE && new_tile) {       // finish item j-1 with its own tile's cos / sin before they are replaced
            __syncthreads();                           // its (rrms, coef)
            if (pend_active) sweep2(pend_s, pend_buf, pend_b, pend_h, pend_t);
            pend = false;
            flushed = true;
        }
        if (ROPE && new_tile && active) load_table(t);
        if (!mbar_wait_bounded(&full[s], (uint32_t)(j / NST) & 1u, test.wait_limit)) atomicExch(&give_up, 1);
        const T *xt = reinterpret_cast<const T *>(stages + (size_t)s * STAGE_BYTES);
        T *dt = reinterpret_cast<T *>(stages + (size_t)s * STAGE_BYTES + TILE_BYTES);
        if (GQ > 1) {       // head sum into the first dy tile; a thread only ever touches its own entries of the tiles
#pragma unroll
            for (int k = 0; k < RPT; k++) {
                const int e = (rg * RPT + k) * TW + lg * VEC;
                Raw<T, VEC> a;
                a.load(dt + e);
                V<VEC> acc = a.get();
#pragma unroll
                for (int r = 1; r < GQ; r++) {
                    Raw<T, VEC> c;
                    c.load(dt + (size_t)r * (TILE_BYTES / sizeof(T)) + e);
                    acc = vadd(acc, c.get());
                }
                a.put(acc);
                a.store(dt + e);
            }
        }
        V<VEC> ss = V<VEC>::splat(0.0f), dot = V<VEC>::splat(0.0f);
#pragma unroll
        for (int p = 0; p < RPT / 2; p++) {
            V<VEC> x0, x1, g0, g1;
            load_pair(xt, dt, p, x0, x1, g0, g1);
            ss = vfma(x0, x0, ss);
            ss = vfma(x1, x1, ss);
            dot = vfma_s(vmul(g0, x0), wc[2 * p], dot);
            dot = vfma_s(vmul(g1, x1), wc[2 * p + 1], dot);
        }
        ss = warp_rowgroup_sum<VEC, QK_LG>(ss);
        dot = warp_rowgroup_sum<VEC, QK_LG>(dot);
        if ((threadIdx.x & 31) < QK_LG) {
            lanes_to_smem<VEC>(&red[buf][0][threadIdx.x >> 5][lg * VEC], ss);
            lanes_to_smem<VEC>(&red[buf][1][threadIdx.x >> 5][lg * VEC], dot);
        }
        __syncthreads();                                   // sweep 1 of item j published; every sweep 2 issued before it is done
        if (*(volatile int *)&give_up) {
            if (threadIdx.x == 0) { atomicAdd(&status->wait_giveups, 1); drain(j); }
            break;
        }
        if (threadIdx.x == 0) {
            // PIPE: sweep 2 of item j-1 runs after this barrier, so items <= j-2 are done (item j-1 too when it was flushed);
            // otherwise sweep 2 of item j-1 ran before this barrier
            freed = PIPE ? (flushed ? j - 1 : j - 2) : j - 1;
            if (next_issue < n_items && next_issue - NST <= freed) { fence_proxy_async(); }
            while (next_issue < n_items && next_issue - NST <= freed) issue(next_issue++);
        }
        {
            constexpr int P = QK_THREADS / TW;
            const float s0 = block_column_sum<NWARP, TW, QK_THREADS>(&red[buf][0][0][0], threadIdx.x);
            const float s1 = block_column_sum<NWARP, TW, QK_THREADS>(&red[buf][1][0][0], threadIdx.x);
            if (threadIdx.x % P == 0) {
                const float r1 = 1.0f / sqrtf(__fadd_rn(__fmul_rn(s0, invd), eps));
                float r2 = r1 * r1;
                r2 = r2 * invd;
                tot[buf][0][threadIdx.x / P] = r1;
                tot[buf][1][threadIdx.x / P] = s1 * r2;
            }
        }
        if (PIPE) {
            if (pend && pend_active) sweep2(pend_s, pend_buf, pend_b, pend_h, pend_t);      // item j-1 (same token tile: same cos / sin)
            pend = true; pend_s = s; pend_buf = buf; pend_b = b; pend_h = h; pend_t = t; pend_active = active;
        } else {
            __syncthreads();
            if (active) sweep2(s, buf, b, h, t);
        }
    }
    if (PIPE && pend && !*(volatile int *)&give_up) {
        __syncthreads();                                   // the (rrms, coef) of the last item
        if (pend_active) sweep2(pend_s, pend_buf, pend_b, pend_h, pend_t);
    }
#pragma unroll
    for (int k = 0; k < RPT; k++) {
        float sum = dwacc[k];
#pragma unroll
        for (int off = QK_LG / 2; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if (lg == 0) partial[(size_t)blockIdx.x * HD + rg * RPT + k] = sum;
    }
}

// ------------------------------------------------------------------ fused kernels, any head width
// One thread per (sequence, head, token), scalar loads that coalesce along S.  Used for head
// widths and alignments the register-resident kernels above do not cover; same arithmetic, so a
// result does not depend on which path ran (a single rounding to the storage type at the end).
constexpr int QKG_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(QKG_THREADS)
qk_rope_fwd_generic_kernel(T *__restrict__ out, const T *__restrict__ x, const float *__restrict__ w, int hd, int S,
                           long long total, float eps, int pos0, const __grid_constant__ RopeFreq freq) {
    const long long idx = (long long)blockIdx.x * QKG_THREADS + threadIdx.x;
    if (idx >= total) return;
    const int t = (int)(idx % S);
    const size_t base = (size_t)(idx / S) * hd * S + t;
    float ss = 0.0f;
    for (int c = 0; c < hd; c++) { const float v = Elt<T>::to_f(x[base + (size_t)c * S]); ss += v * v; }
    const float rr = 1.0f / sqrtf(__fadd_rn(__fmul_rn(ss, 1.0f / (float)hd), eps));
    for (int i = 0; i < hd / 2; i++) {
        const float theta = (float)(pos0 + t) * freq.f[i];
        const float cs = cosf(theta), sn = sinf(theta);
        const float a = (Elt<T>::to_f(x[base + (size_t)(2 * i) * S]) * rr) * __ldg(w + 2 * i);
        const float b = (Elt<T>::to_f(x[base + (size_t)(2 * i + 1) * S]) * rr) * __ldg(w + 2 * i + 1);
        out[base + (size_t)(2 * i) * S] = Elt<T>::from_f(__fsub_rn(__fmul_rn(a, cs), __fmul_rn(b, sn)));
        out[base + (size_t)(2 * i + 1) * S] = Elt<T>::from_f(__fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, cs)));
    }
}

__device__ __forceinline__ float block_sum_128(float v, float *sh) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    return (sh[0] + sh[1]) + (sh[2] + sh[3]);
}

template <typename T>
__global__ void __launch_bounds__(QKG_THREADS)
qk_rope_bwd_generic_kernel(T *__restrict__ dx, float *__restrict__ partial, const T *__restrict__ dy,
                           const T *__restrict__ x, const float *__restrict__ w, int hd, int S, long long total,
                           float eps, int pos0, unsigned flags, const __grid_constant__ RopeFreq freq) {
    __shared__ float dwacc[256];
    __shared__ float sh[4];
    const bool exact = (flags & ANE_NORM_BWD_EXACT) != 0;
    const float invd = 1.0f / (float)hd;
    for (int c = threadIdx.x; c < hd; c += QKG_THREADS) dwacc[c] = 0.0f;
    __syncthreads();
    for (long long blk = (long long)blockIdx.x * QKG_THREADS; blk < total; blk += (long long)gridDim.x * QKG_THREADS) {
        const long long idx = blk + threadIdx.x;
        const bool valid = idx < total;
        const int t = valid ? (int)(idx % S) : 0;
        const size_t base = valid ? (size_t)(idx / S) * hd * S + t : 0;
        float ss = 0.0f, dot = 0.0f;
        if (valid) {
            for (int i = 0; i < hd / 2; i++) {
                const float theta = (float)(pos0 + t) * freq.f[i];
                const float cs = cosf(theta), sn = sinf(theta);
                const float a = Elt<T>::to_f(dy[base + (size_t)(2 * i) * S]), b = Elt<T>::to_f(dy[base + (size_t)(2 * i + 1) * S]);
                const float g0 = __fadd_rn(__fmul_rn(a, cs), __fmul_rn(b, sn));
                const float g1 = __fadd_rn(__fmul_rn(-a, sn), __fmul_rn(b, cs));
                const float x0 = Elt<T>::to_f(x[base + (size_t)(2 * i) * S]), x1 = Elt<T>::to_f(x[base + (size_t)(2 * i + 1) * S]);
                ss += x0 * x0; ss += x1 * x1;
                dot += (g0 * x0) * __ldg(w + 2 * i);
                dot += (g1 * x1) * __ldg(w + 2 * i + 1);
            }
        }
        const float rr = 1.0f / sqrtf(__fadd_rn(__fmul_rn(ss, invd), eps));
        float r2 = rr * rr;
        r2 = r2 * invd;
        const float coef = dot * r2;
        for (int i = 0; i < hd / 2; i++) {
            float dwp[2] = {0.0f, 0.0f};
            if (valid) {
                const float theta = (float)(pos0 + t) * freq.f[i];
                const float cs = cosf(theta), sn = sinf(theta);
                const float a = Elt<T>::to_f(dy[base + (size_t)(2 * i) * S]), b = Elt<T>::to_f(dy[base + (size_t)(2 * i + 1) * S]);
                float g[2];
                g[0] = __fadd_rn(__fmul_rn(a, cs), __fmul_rn(b, sn));
                g[1] = __fadd_rn(__fmul_rn(-a, sn), __fmul_rn(b, cs));
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    const int c = 2 * i + k;
                    const float xv = Elt<T>::to_f(x[base + (size_t)c * S]);
                    const float wc = __ldg(w + c);
                    float o;
                    if (exact) {
                        o = __fmul_rn(__fsub_rn(__fmul_rn(g[k], wc), __fmul_rn(xv, coef)), rr);
                    } else {
                        float tmp = __fmul_rn(xv, coef);
                        tmp = __fsub_rn(g[k], tmp);
                        tmp = tmp * rr;
                        o = tmp * wc;
                    }
                    dx[base + (size_t)c * S] = Elt<T>::from_f(o);
                    dwp[k] = (g[k] * xv) * rr;
                }
            }
            const float s0 = block_sum_128(dwp[0], sh);
            const float s1 = block_sum_128(dwp[1], sh);
            if (threadIdx.x == 0) { dwacc[2 * i] += s0; dwacc[2 * i + 1] += s1; }
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < hd; c += QKG_THREADS) partial[(size_t)blockIdx.x * hd + c] = dwacc[c];
}

template <typename T>
static int launch_qk_rope_fwd_generic(cudaStream_t st, int B, int heads, int hd, int S, void *out, const void *x,
                                      const float *w, float eps, int pos0, const RopeFreq &fq) {
    const long long total = (long long)B * heads * S;
    const long long blocks = (total + QKG_THREADS - 1) / QKG_THREADS;
    qk_rope_fwd_generic_kernel<T><<<(unsigned)blocks, QKG_THREADS, 0, st>>>((T *)out, (const T *)x, w, hd, S, total, eps, pos0, fq);
    ANE_LAUNCH_OK(1);
    return ANE_CUDA_OK;
}

template <typename T>
static int launch_qk_rope_bwd_generic(cudaStream_t st, int B, int heads, int hd, int S, void *dx, float *dw, const void *dy,
                                      const void *x, const float *w, float eps, int pos0, unsigned flags, const RopeFreq &fq) {
    const long long total = (long long)B * heads * S;
    long long blocks = (total + QKG_THREADS - 1) / QKG_THREADS;
    const long long cap = (long long)ctx().sm_count * 8;
    if (blocks > cap) blocks = cap;
    float *partial = static_cast<float *>(workspace((size_t)blocks * hd * sizeof(float)));
    if (!partial) return fail(ANE_CUDA_ERR_NOMEM, "rope_qknorm_bwd: no scratch");
    qk_rope_bwd_generic_kernel<T><<<(unsigned)blocks, QKG_THREADS, 0, st>>>((T *)dx, partial, (const T *)dy, (const T *)x, w, hd, S,
                                                                           total, eps, pos0, flags, fq);
    column_sum_add_kernel<><<<(hd + 31) / 32, 256, 0, st>>>(dw, partial, (int)blocks, hd);
    ANE_LAUNCH_OK(2);
    return ANE_CUDA_OK;
}

static RingTest ring_test() {
    RingTest t;
    t.skip_item = tuning("qk_test_skip_item", -1);
    const int lim = tuning("qk_wait_limit", 0);
    t.wait_limit = lim > 0 ? (uint32_t)lim : MBAR_WAIT_LIMIT;
    return t;
}

// RoPE^-1 + QK-norm backward with the grouped-query head sum folded in (two-stage ring: a stage holds the x tile and
// `ratio` dy tiles).
template <typename T>
static int launch_qk_bwd_gqa(cudaStream_t st, int B, int heads, int ratio, int hd, int S, void *dx, float *dw, const void *dy,
                             const void *x, const float *w, float eps, float base, int pos0, unsigned flags, const RopeFreq &fq) {
    constexpr int VEC = Elt<T>::VEC;
    int trc = ANE_CUDA_OK;
    const float *cosT = rope_table(st, hd, S, base, pos0, fq, &trc, "rope_qknorm_bwd_gqa");
    if (!cosT) return trc;
    const float *sinT = cosT + (size_t)S * (hd / 2);
    const int tps = (S + QK_LG * VEC - 1) / (QK_LG * VEC);
    const int ntiles = B * tps;
    const ane_dtype dte = sizeof(T) == 4 ? ANE_F32 : (std::is_same<T, __half>::value ? ANE_F16 : ANE_BF16);
    CUtensorMap xmap, dymap;
    if (int rc = make_bcs_tensor_map(&xmap, dte, x, B, heads * hd, S, QK_LG * VEC, hd)) return rc;
    if (int rc = make_bcs_tensor_map(&dymap, dte, dy, B, heads * ratio * hd, S, QK_LG * VEC, hd)) return rc;
    int grid = 0;
    float *partial = nullptr;
#define ANE_QKB_GQA(RPTv, GQv)                                                                                       \
    do {                                                                                                             \
        auto k = qk_bwd_tma_kernel<T, RPTv, true, 2, GQv>;                                                            \
        const size_t smem = (size_t)2 * (1 + GQv) * (RPTv * QK_R) * (QK_LG * VEC) * sizeof(T) + 128;                    \
        ANE_CUDA_TRY(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));               \
        int per_sm = 0;                                                                                              \
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, QK_THREADS, smem) != cudaSuccess || per_sm < 1) per_sm = 1; \
        grid = per_sm * ctx().sm_count;                                                                              \
        if (grid > ntiles) grid = ntiles;                                                                            \
        partial = static_cast<float *>(workspace((size_t)grid * hd * sizeof(float)));                                \
        if (!partial) return fail(ANE_CUDA_ERR_NOMEM, "rope_qknorm_bwd_gqa: no scratch");                            \
        launch_dep(DEP_QK, k, dim3((unsigned)grid), dim3(QK_THREADS), smem, st, (T *)dx, partial, dymap, xmap, w, heads, S, tps, ntiles, eps, flags, ctx().status, cosT, sinT, ring_test()); \
    } while (0)
    if (hd == 128) { if (ratio == 2) ANE_QKB_GQA(4, 2); else ANE_QKB_GQA(4, 4); }
    else { if (ratio == 2) ANE_QKB_GQA(2, 2); else ANE_QKB_GQA(2, 4); }
#undef ANE_QKB_GQA
    launch_dep(DEP_COLSUM, column_sum_add_kernel<>, dim3((hd + 31) / 32), dim3(256), 0, st, dw, (const float *)partial, grid, hd);
    ANE_LAUNCH_OK(2);
    return ANE_CUDA_OK;
}

static int fill_freq(RopeFreq &fq, int hd, float base) {
    if (hd < 2 || (hd & 1) || hd > 256) return fail(ANE_CUDA_ERR_UNSUPPORTED, "rope: head dim %d must be even and <= 256", hd);
    // freq = 1/powf(base, 2*i/hd) with the host libm                    cpu_ops.h:172
    for (int i = 0; i < hd / 2; i++) fq.f[i] = 1.0f / powf(base, 2.0f * i / (float)hd);
    for (int i = hd / 2; i < 128; i++) fq.f[i] = 0.0f;
    return ANE_CUDA_OK;
}

template <typename T>
static int launch_rope(cudaStream_t st, int B, int heads, int hd, int S, void *out, const void *x, float base, int pos0, bool inverse,
                       const RopeFreq &fq) {
    constexpr int VEC = Elt<T>::VEC;
    const bool vec = (S % VEC == 0) && aligned16(out) && aligned16(x);
    if (vec) {
        // the cached table when it exists or can be made now; a miss while the stream is being captured, or after
        // ane_cuda_freeze, falls back to the in-kernel evaluation (same bits) instead of failing
        int trc = ANE_CUDA_OK;
        const float *cosT = tuning("rope_table", 1) ? rope_table(st, hd, S, base, pos0, fq, &trc, "rope") : nullptr;
        const float *sinT = cosT ? cosT + (size_t)S * (hd / 2) : nullptr;
#define ANE_ROPE_LG(LGv)                                                                                             \
        do {                                                                                                         \
            const int tps_ = (S + (LGv) * VEC - 1) / ((LGv) * VEC);                                                   \
            dim3 grid_((unsigned)(B * tps_), (unsigned)((hd / 2 + (QK_THREADS / (LGv)) - 1) / (QK_THREADS / (LGv)))); \
            rope_kernel<T, VEC, LGv><<<grid_, QK_THREADS, 0, st>>>((T *)out, (const T *)x, heads, hd, S, tps_, pos0, inverse, fq, cosT, sinT); \
        } while (0)
        switch (tuning("rope_lg", 16)) {
            case 32: ANE_ROPE_LG(32); break;
            case 16: ANE_ROPE_LG(16); break;
            default: ANE_ROPE_LG(8); break;
        }
#undef ANE_ROPE_LG
    } else {
        constexpr int LG = 32;
        const int tps = (S + LG - 1) / LG;
        dim3 grid((unsigned)(B * tps), (unsigned)((hd / 2 + (QK_THREADS / LG) - 1) / (QK_THREADS / LG)));
        rope_kernel<T, 1, LG><<<grid, QK_THREADS, 0, st>>>((T *)out, (const T *)x, heads, hd, S, tps, pos0, inverse, fq, nullptr, nullptr);
    }
    ANE_LAUNCH_OK(1);
    return ANE_CUDA_OK;
}

template <typename KernelT>
static int qk_persistent_grid(KernelT kernel, int ntiles) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, QK_THREADS, 0) != cudaSuccess || per_sm < 1) per_sm = 1;
    long g = (long)per_sm * ctx().sm_count;
    if (g > ntiles) g = ntiles;
    if (g < 1) g = 1;
    return (int)g;
}

// Q and K of one layer side by side (the *_pair entry points): the two launches of the ring kernel run at the same time,
// on the caller's stream and on a stream of the library, each on its share of the persistent grid (16 : 8 heads -> two
// thirds and one third of the blocks), so the pair pays one ramp and one tail instead of two.  The shares add up to no more
// than the blocks that are resident at once: neither launch waits for a second wave.
struct QkShare { int num = 1, den = 1; float *partial = nullptr; };
static QkShare g_share;      // set by the pair entry points around the launches they make (one host thread at a time)
static inline int share_grid(int g) {
    const long long s = (long long)g * g_share.num / g_share.den;
    return s < 1 ? 1 : (int)s;
}
struct QkSide { cudaStream_t stream = nullptr; cudaEvent_t fork = nullptr, join = nullptr; bool ok = false; };
static QkSide g_qk_side;
static QkSide *qk_side() {
    if (g_qk_side.ok) return &g_qk_side;
    if (cudaStreamCreateWithFlags(&g_qk_side.stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&g_qk_side.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&g_qk_side.join, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    g_qk_side.ok = true;
    return &g_qk_side;
}
void qk_side_release() {
    if (g_qk_side.stream) cudaStreamDestroy(g_qk_side.stream);
    if (g_qk_side.fork) cudaEventDestroy(g_qk_side.fork);
    if (g_qk_side.join) cudaEventDestroy(g_qk_side.join);
    g_qk_side = QkSide();
}

template <typename T, bool ROPE>
static bool qk_fast_ok(int hd, int S, const void *a, const void *b, const void *c) {
    constexpr int VEC = Elt<T>::VEC;
    return (hd == 128 || hd == 64) && (S % VEC == 0) && aligned16(a) && aligned16(b) && (!c || aligned16(c));
}

template <typename T, bool ROPE>
static int launch_qk_fwd(cudaStream_t st, int B, int heads, int hd, int S, void *out, const void *x, const float *w,
                         float eps, float base, int pos0, const RopeFreq &fq, int out_ratio = 1) {
    constexpr int VEC = Elt<T>::VEC;
    const float *cosT = nullptr, *sinT = nullptr;
    if (ROPE) {
        int trc = ANE_CUDA_OK;
        cosT = rope_table(st, hd, S, base, pos0, fq, &trc, "qknorm_rope");
        if (!cosT) return trc;
        sinT = cosT + (size_t)S * (hd / 2);
    }
    const int tps = (S + QK_LG * VEC - 1) / (QK_LG * VEC);
    const unsigned grid = (unsigned)(B * tps);
    const int hb = out_ratio > 1 ? 3 : tuning("qk_fwd", 3);       // the tiled output exists in the TMA kernel only
    if (hb >= 3) {       // TMA-fed ring of hb stages
        CUtensorMap xmap;
        if (int rc = make_bcs_tensor_map(&xmap, sizeof(T) == 4 ? ANE_F32 : (std::is_same<T, __half>::value ? ANE_F16 : ANE_BF16), x, B,
                                         heads * hd, S, QK_LG * VEC, hd)) return rc;
        const int ntiles = B * tps;
        const bool pipe = tuning("qk_fwd_pipe", 1) != 0;      // one barrier per item (default) or two
#define ANE_QKF_TMA(RPTv, NSTv)                                                                                      \
        do {                                                                                                         \
            auto k = out_ratio > 1 ? (pipe ? qk_fwd_tma_kernel<T, RPTv, ROPE, NSTv, true, true> : qk_fwd_tma_kernel<T, RPTv, ROPE, NSTv, true, false>) \
                                   : (pipe ? qk_fwd_tma_kernel<T, RPTv, ROPE, NSTv, false, true> : qk_fwd_tma_kernel<T, RPTv, ROPE, NSTv, false, false>); \
            const size_t smem = (size_t)NSTv * (RPTv * QK_R) * (QK_LG * VEC) * sizeof(T) + 128;                             \
            ANE_CUDA_TRY(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));           \
            int per_sm = 0;                                                                                          \
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, QK_THREADS, smem) != cudaSuccess || per_sm < 1) per_sm = 1; \
            int g = share_grid(per_sm * ctx().sm_count);                                                             \
            if (g > ntiles) g = ntiles;                                                                              \
            launch_dep(DEP_QK, k, dim3((unsigned)g), dim3(QK_THREADS), smem, st, (T *)out, xmap, w, heads, S, tps, ntiles, eps, ctx().status, cosT, sinT, out_ratio, ring_test()); \
        } while (0)
        if (hd == 128) { if (hb == 3) ANE_QKF_TMA(4, 3); else if (hb == 4) ANE_QKF_TMA(4, 4); else ANE_QKF_TMA(4, 6); }
        else { if (hb == 3) ANE_QKF_TMA(2, 3); else if (hb == 4) ANE_QKF_TMA(2, 4); else ANE_QKF_TMA(2, 6); }
#undef ANE_QKF_TMA
        ANE_LAUNCH_OK(1);
        return ANE_CUDA_OK;
    }
#define ANE_QKF(RPTv, HBv) qk_fwd_kernel<T, RPTv, ROPE, HBv><<<grid, QK_THREADS, 0, st>>>((T *)out, (const T *)x, w, heads, S, tps, eps, cosT, sinT)
    if (hd == 128) { if (hb == 1) ANE_QKF(4, 1); else ANE_QKF(4, 2); }
    else { if (hb == 1) ANE_QKF(2, 1); else ANE_QKF(2, 2); }
#undef ANE_QKF
    ANE_LAUNCH_OK(1);
    return ANE_CUDA_OK;
}

template <typename T, bool ROPE>
static int launch_qk_bwd(cudaStream_t st, int B, int heads, int hd, int S, void *dx, float *dw, const void *dy,
                         const void *x, const float *w, float eps, float base, int pos0, unsigned flags, const RopeFreq &fq) {
    constexpr int VEC = Elt<T>::VEC;
    const float *cosT = nullptr, *sinT = nullptr;
    if (ROPE) {
        int trc = ANE_CUDA_OK;
        cosT = rope_table(st, hd, S, base, pos0, fq, &trc, "rope_qknorm_bwd");
        if (!cosT) return trc;
        sinT = cosT + (size_t)S * (hd / 2);
    }
    const int tps = (S + QK_LG * VEC - 1) / (QK_LG * VEC);
    const int ntiles = B * tps;
    const int hb = tuning("qk_bwd", 3);
    int grid = 0;
    float *partial = nullptr;
    if (hb >= 3) {       // TMA-fed ring of hb stages
        const ane_dtype dte = sizeof(T) == 4 ? ANE_F32 : (std::is_same<T, __half>::value ? ANE_F16 : ANE_BF16);
        CUtensorMap xmap, dymap;
        if (int rc = make_bcs_tensor_map(&xmap, dte, x, B, heads * hd, S, QK_LG * VEC, hd)) return rc;
        if (int rc = make_bcs_tensor_map(&dymap, dte, dy, B, heads * hd, S, QK_LG * VEC, hd)) return rc;
        const bool pipe_b = tuning("qk_bwd_pipe", ANE_QK_BWD_PIPE_DEFAULT) != 0;      // one barrier per item, or two
#define ANE_QKB_TMA(RPTv, NSTv)                                                                                      \
        do {                                                                                                         \
            auto k = pipe_b ? qk_bwd_tma_kernel<T, RPTv, ROPE, NSTv, 1, true> : qk_bwd_tma_kernel<T, RPTv, ROPE, NSTv, 1, false>; \
            const size_t smem = (size_t)NSTv * 2 * (RPTv * QK_R) * (QK_LG * VEC) * sizeof(T) + 128;                         \
            ANE_CUDA_TRY(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));           \
            int per_sm = 0;                                                                                          \
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, QK_THREADS, smem) != cudaSuccess || per_sm < 1) per_sm = 1; \
            grid = share_grid(per_sm * ctx().sm_count);                                                              \
            if (grid > ntiles) grid = ntiles;                                                                        \
            partial = g_share.partial ? g_share.partial : static_cast<float *>(workspace((size_t)grid * hd * sizeof(float))); \
            if (!partial) return fail(ANE_CUDA_ERR_NOMEM, "qknorm_bwd: no scratch");                                 \
            launch_dep(DEP_QK, k, dim3((unsigned)grid), dim3(QK_THREADS), smem, st, (T *)dx, partial, dymap, xmap, w, heads, S, tps, ntiles, eps, flags, ctx().status, cosT, sinT, ring_test()); \
        } while (0)
        if (hd == 128) { if (hb == 3) ANE_QKB_TMA(4, 3); else ANE_QKB_TMA(4, 4); }
        else { if (hb == 3) ANE_QKB_TMA(2, 3); else ANE_QKB_TMA(2, 4); }
#undef ANE_QKB_TMA
        launch_dep(DEP_COLSUM, column_sum_add_kernel<>, dim3((hd + 31) / 32), dim3(256), 0, st, dw, (const float *)partial, grid, hd);
        ANE_LAUNCH_OK(2);
        return ANE_CUDA_OK;
    }
#define ANE_QKB(RPTv, HBv)                                                                                          \
    do {                                                                                                            \
        auto k = qk_bwd_kernel<T, RPTv, ROPE, HBv>;                                                                  \
        grid = qk_persistent_grid(k, ntiles);                                                                       \
        partial = static_cast<float *>(workspace((size_t)grid * hd * sizeof(float)));                               \
        if (!partial) return fail(ANE_CUDA_ERR_NOMEM, "qknorm_bwd: no scratch");                                    \
        k<<<grid, QK_THREADS, 0, st>>>((T *)dx, partial, (const T *)dy, (const T *)x, w, heads, S, tps, ntiles, eps, flags, cosT, sinT); \
    } while (0)
    (void)hb;       // one head per step: two would need more than 48 KiB of static shared memory
    if (hd == 128) ANE_QKB(4, 1);
    else ANE_QKB(2, 1);
#undef ANE_QKB
    column_sum_add_kernel<><<<(hd + 31) / 32, 256, 0, st>>>(dw, partial, grid, hd);
    ANE_LAUNCH_OK(2);
    return ANE_CUDA_OK;
}

static int check_qk(const char *fn, int B, int heads, int hd, int S) {
    if (B < 1 || heads < 1 || hd < 1 || S < 1)
        return fail(ANE_CUDA_ERR_INVALID, "%s: B, heads, hd, S must be positive (got %d, %d, %d, %d)", fn, B, heads, hd, S);
    if ((long long)B * heads > 0x7fffffLL || (long long)B * ((S + 7) / 8) > 0x7fffffffLL)
        return fail(ANE_CUDA_ERR_UNSUPPORTED, "%s: shape too large", fn);
    return ANE_CUDA_OK;
}

}  // namespace ane

using namespace ane;

extern "C" {

int ane_cuda_rope_dev(void *stream, ane_dtype dtype, int B, int C, int S, int hd, void *out, const void *x, float base,
                      int pos0, unsigned flags) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && x, "%s: null pointer", __func__);
    ANE_REQUIRE(dtype_ok(dtype), "%s: bad dtype", __func__);
    ANE_REQUIRE(B >= 1 && C >= 1 && S >= 1 && hd >= 2 && C % hd == 0, "%s: bad shape B=%d C=%d S=%d hd=%d", __func__, B, C, S, hd);
    ANE_REQUIRE(flags == ANE_ROPE_FORWARD || flags == ANE_ROPE_INVERSE, "%s: bad flags %u", __func__, flags);
    ANE_CHECK_EXTENT(out, (size_t)B * C * S * dtype_size(dtype)); ANE_CHECK_EXTENT(x, (size_t)B * C * S * dtype_size(dtype));
    RopeFreq fq;
    if (int rc = fill_freq(fq, hd, base)) return rc;
    ANE_DISPATCH_DTYPE(dtype, T, return (launch_rope<T>((cudaStream_t)stream, B, C / hd, hd, S, out, x, base, pos0, flags == ANE_ROPE_INVERSE, fq)));
    return ANE_CUDA_OK;
}

int ane_cuda_qknorm_dev(void *stream, ane_dtype dtype, int B, int heads, int hd, int S, void *out, const void *x,
                        const float *w, float eps) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && x && w, "%s: null pointer", __func__);
    ANE_REQUIRE(dtype_ok(dtype), "%s: bad dtype", __func__);
    if (int rc = check_qk(__func__, B, heads, hd, S)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    {
        const size_t nb = (size_t)B * heads * hd * S * dtype_size(dtype);
        ANE_CHECK_EXTENT(out, nb); ANE_CHECK_EXTENT(x, nb);
        ANE_CHECK_EXTENT(w, (size_t)hd * 4);
    }
    RopeFreq fq = {};
    ANE_DISPATCH_DTYPE(dtype, T,
        if (qk_fast_ok<T, false>(hd, S, out, x, nullptr)) return (launch_qk_fwd<T, false>(st, B, heads, hd, S, out, x, w, eps, 0.0f, 0, fq)));
    return rmsnorm_fwd_any(st, dtype, B * heads, hd, S, out, x, w, eps);
}

int ane_cuda_qknorm_bwd_dev(void *stream, ane_dtype dtype, int B, int heads, int hd, int S, void *dx, float *dw,
                            const void *dy, const void *x, const float *w, float eps, unsigned flags) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dx && dw && dy && x && w, "%s: null pointer", __func__);
    ANE_REQUIRE(dtype_ok(dtype), "%s: bad dtype", __func__);
    ANE_REQUIRE(flags == ANE_NORM_BWD_REFERENCE || flags == ANE_NORM_BWD_EXACT, "%s: bad flags %u", __func__, flags);
    if (int rc = check_qk(__func__, B, heads, hd, S)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    {
        const size_t nb = (size_t)B * heads * hd * S * dtype_size(dtype);
        ANE_CHECK_EXTENT(dx, nb); ANE_CHECK_EXTENT(dy, nb); ANE_CHECK_EXTENT(x, nb);
        ANE_CHECK_EXTENT(w, (size_t)hd * 4); ANE_CHECK_EXTENT(dw, (size_t)hd * 4);
    }
    RopeFreq fq = {};
    ANE_DISPATCH_DTYPE(dtype, T,
        if (qk_fast_ok<T, false>(hd, S, dx, dy, x)) return (launch_qk_bwd<T, false>(st, B, heads, hd, S, dx, dw, dy, x, w, eps, 0.0f, 0, flags, fq)));
    return rmsnorm_bwd_any(st, dtype, B * heads, hd, S, dx, dw, dy, x, w, nullptr, eps, flags);
}

int ane_cuda_qknorm_rope_dev(void *stream, ane_dtype dtype, int B, int heads, int hd, int S, void *out, const void *x,
                             const float *w, float eps, float base, int pos0) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out && x && w, "%s: null pointer", __func__);
    ANE_REQUIRE(dtype_ok(dtype), "%s: bad dtype", __func__);
    if (int rc = check_qk(__func__, B, heads, hd, S)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    {
        const size_t nb = (size_t)B * heads * hd * S * dtype_size(dtype);
        ANE_CHECK_EXTENT(out, nb); ANE_CHECK_EXTENT(x, nb);
        ANE_CHECK_EXTENT(w, (size_t)hd * 4);
    }
    RopeFreq fq;
    if (int rc = fill_freq(fq, hd, base)) return rc;
    ANE_DISPATCH_DTYPE(dtype, T,
        if (qk_fast_ok<T, true>(hd, S, out, x, nullptr)) return (launch_qk_fwd<T, true>(st, B, heads, hd, S, out, x, w, eps, base, pos0, fq)));
    // other head widths and unaligned shapes
    ANE_DISPATCH_DTYPE(dtype, T, return (launch_qk_rope_fwd_generic<T>(st, B, heads, hd, S, out, x, w, eps, pos0, fq)));
    return ANE_CUDA_OK;
}

int ane_cuda_qknorm_rope_tiled_dev(void *stream, ane_dtype dtype, int B, int kv_heads, int ratio, int hd, int S, void *out_tiled,
                                   const void *x, const float *w, float eps, float base, int pos0) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out_tiled && x && w, "%s: null pointer", __func__);
    ANE_REQUIRE(dtype_ok(dtype), "%s: bad dtype", __func__);
    ANE_REQUIRE(ratio >= 1 && ratio <= 64, "%s: bad ratio %d", __func__, ratio);
    if (int rc = check_qk(__func__, B, kv_heads, hd, S)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    RopeFreq fq;
    if (int rc = fill_freq(fq, hd, base)) return rc;
    ANE_DISPATCH_DTYPE(dtype, T,
        if (qk_fast_ok<T, true>(hd, S, out_tiled, x, nullptr))
            return (launch_qk_fwd<T, true>(st, B, kv_heads, hd, S, out_tiled, x, w, eps, base, pos0, fq, ratio)));
    return fail(ANE_CUDA_ERR_UNSUPPORTED, "%s: the tiled output covers head widths 64 and 128 and 16-byte aligned rows; use "
                "ane_cuda_qknorm_rope_dev followed by ane_cuda_gqa_tile_dev for other shapes", __func__);
}

int ane_cuda_rope_qknorm_bwd_gqa_dev(void *stream, ane_dtype dtype, int B, int kv_heads, int ratio, int hd, int S, void *dx, float *dw,
                                     const void *dy_tiled, const void *x, const float *w, float eps, float base, int pos0,
                                     unsigned flags) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dx && dw && dy_tiled && x && w, "%s: null pointer", __func__);
    ANE_REQUIRE(dtype_ok(dtype), "%s: bad dtype", __func__);
    ANE_REQUIRE(flags == ANE_NORM_BWD_REFERENCE || flags == ANE_NORM_BWD_EXACT, "%s: bad flags %u", __func__, flags);
    if (int rc = check_qk(__func__, B, kv_heads, hd, S)) return rc;
    if (ratio == 1) return ane_cuda_rope_qknorm_bwd_dev(stream, dtype, B, kv_heads, hd, S, dx, dw, dy_tiled, x, w, eps, base, pos0, flags);
    cudaStream_t st = (cudaStream_t)stream;
    RopeFreq fq;
    if (int rc = fill_freq(fq, hd, base)) return rc;
    ANE_DISPATCH_DTYPE(dtype, T,
        if ((ratio == 2 || ratio == 4) && qk_fast_ok<T, true>(hd, S, dx, dy_tiled, x))
            return (launch_qk_bwd_gqa<T>(st, B, kv_heads, ratio, hd, S, dx, dw, dy_tiled, x, w, eps, base, pos0, flags, fq)));
    return fail(ANE_CUDA_ERR_UNSUPPORTED, "%s: the fused form covers ratios 2 and 4, head widths 64 and 128 and 16-byte aligned rows; "
                "use ane_cuda_gqa_reduce_dev followed by ane_cuda_rope_qknorm_bwd_dev for other shapes", __func__);
}

int ane_cuda_rope_qknorm_bwd_dev(void *stream, ane_dtype dtype, int B, int heads, int hd, int S, void *dx, float *dw,
                                 const void *dy, const void *x, const float *w, float eps, float base, int pos0,
                                 unsigned flags) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dx && dw && dy && x && w, "%s: null pointer", __func__);
    ANE_REQUIRE(dtype_ok(dtype), "%s: bad dtype", __func__);
    ANE_REQUIRE(flags == ANE_NORM_BWD_REFERENCE || flags == ANE_NORM_BWD_EXACT, "%s: bad flags %u", __func__, flags);
    if (int rc = check_qk(__func__, B, heads, hd, S)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    {
        const size_t nb = (size_t)B * heads * hd * S * dtype_size(dtype);
        ANE_CHECK_EXTENT(dx, nb); ANE_CHECK_EXTENT(dy, nb); ANE_CHECK_EXTENT(x, nb);
        ANE_CHECK_EXTENT(w, (size_t)hd * 4); ANE_CHECK_EXTENT(dw, (size_t)hd * 4);
    }
    RopeFreq fq;
    if (int rc = fill_freq(fq, hd, base)) return rc;
    ANE_DISPATCH_DTYPE(dtype, T,
        if (qk_fast_ok<T, true>(hd, S, dx, dy, x)) return (launch_qk_bwd<T, true>(st, B, heads, hd, S, dx, dw, dy, x, w, eps, base, pos0, flags, fq)));
    // other head widths and unaligned shapes
    ANE_DISPATCH_DTYPE(dtype, T, return (launch_qk_rope_bwd_generic<T>(st, B, heads, hd, S, dx, dw, dy, x, w, eps, pos0, flags, fq)));
    return ANE_CUDA_OK;
}

// ---- Q and K of one layer in one call
static bool pair_side_by_side(ane_dtype dtype, int hd, int S, const char *stage_knob, std::initializer_list<const void *> ptrs) {
    if (tuning("qk_pair", 1) == 0 || tuning(stage_knob, 3) < 3) return false;
    if (!(hd == 128 || hd == 64) || !dtype_ok(dtype) || S % (16 / (int)dtype_size(dtype)) != 0) return false;
    for (const void *p : ptrs)
        if (!aligned16(p)) return false;
    return true;
}

int ane_cuda_qknorm_rope_pair_dev(void *stream, ane_dtype dtype, int B, int heads_q, int heads_k, int hd, int S, void *out_q,
                                  void *out_k, const void *q, const void *k, const float *wq, const float *wk, float eps,
                                  float base, int pos0) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(out_q && out_k && q && k && wq && wk, "%s: null pointer", __func__);
    if (int rc = check_qk(__func__, B, heads_q, hd, S)) return rc;
    if (int rc = check_qk(__func__, B, heads_k, hd, S)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    QkSide *side = pair_side_by_side(dtype, hd, S, "qk_fwd", {out_q, out_k, q, k}) ? qk_side() : nullptr;
    if (!side) {
        if (int rc = ane_cuda_qknorm_rope_dev(stream, dtype, B, heads_q, hd, S, out_q, q, wq, eps, base, pos0)) return rc;
        return ane_cuda_qknorm_rope_dev(stream, dtype, B, heads_k, hd, S, out_k, k, wk, eps, base, pos0);
    }
    ANE_CUDA_TRY(cudaEventRecord(side->fork, st));
    ANE_CUDA_TRY(cudaStreamWaitEvent(side->stream, side->fork, 0));
    g_share = QkShare{heads_q, heads_q + heads_k, nullptr};
    int rc = ane_cuda_qknorm_rope_dev(stream, dtype, B, heads_q, hd, S, out_q, q, wq, eps, base, pos0);
    g_share = QkShare{heads_k, heads_q + heads_k, nullptr};
    const int rc2 = ane_cuda_qknorm_rope_dev(side->stream, dtype, B, heads_k, hd, S, out_k, k, wk, eps, base, pos0);
    g_share = QkShare();
    // the side stream rejoins the caller's stream whatever happened (a capture must not end with a forked stream)
    cudaEventRecord(side->join, side->stream);
    cudaStreamWaitEvent(st, side->join, 0);
    return rc ? rc : rc2;
}

int ane_cuda_rope_qknorm_bwd_pair_dev(void *stream, ane_dtype dtype, int B, int heads_q, int heads_k, int hd, int S, void *dq,
                                      void *dk, float *dwq, float *dwk, const void *dyq, const void *dyk, const void *q,
                                      const void *k, const float *wq, const float *wk, float eps, float base, int pos0,
                                      unsigned flags) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dq && dk && dwq && dwk && dyq && dyk && q && k && wq && wk, "%s: null pointer", __func__);
    if (int rc = check_qk(__func__, B, heads_q, hd, S)) return rc;
    if (int rc = check_qk(__func__, B, heads_k, hd, S)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    QkSide *side = pair_side_by_side(dtype, hd, S, "qk_bwd", {dq, dk, dyq, dyk, q, k}) ? qk_side() : nullptr;
    // one scratch range for both launches' dw partials: they run at the same time
    const size_t rows = (size_t)8 * ctx().sm_count;
    float *partial = side ? static_cast<float *>(workspace(2 * rows * hd * sizeof(float))) : nullptr;
    if (!side || !partial) {
        if (int rc = ane_cuda_rope_qknorm_bwd_dev(stream, dtype, B, heads_q, hd, S, dq, dwq, dyq, q, wq, eps, base, pos0, flags)) return rc;
        return ane_cuda_rope_qknorm_bwd_dev(stream, dtype, B, heads_k, hd, S, dk, dwk, dyk, k, wk, eps, base, pos0, flags);
    }
    ANE_CUDA_TRY(cudaEventRecord(side->fork, st));
    ANE_CUDA_TRY(cudaStreamWaitEvent(side->stream, side->fork, 0));
    g_share = QkShare{heads_q, heads_q + heads_k, partial};
    int rc = ane_cuda_rope_qknorm_bwd_dev(stream, dtype, B, heads_q, hd, S, dq, dwq, dyq, q, wq, eps, base, pos0, flags);
    g_share = QkShare{heads_k, heads_q + heads_k, partial + rows * hd};
    const int rc2 = ane_cuda_rope_qknorm_bwd_dev(side->stream, dtype, B, heads_k, hd, S, dk, dwk, dyk, k, wk, eps, base, pos0, flags);
    g_share = QkShare();
    cudaEventRecord(side->join, side->stream);
    cudaStreamWaitEvent(st, side->join, 0);
    return rc ? rc : rc2;
}

}  // extern "C"
