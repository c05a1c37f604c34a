// embed.cu -- token-embedding gather (a transposing copy) and its scatter-add gradient.
//
// Gather: x[b][d][t] = table[tok[b][t]][d].  Table rows are contiguous along d, x is
// contiguous along t, so a block moves a [tokens x dims] tile through shared memory: row
// chunks are read with consecutive lanes along d, columns are written with consecutive lanes
// along t.  The copy is bit-exact (elements are moved as raw 16- or 32-bit words).
//
// Scatter-add: d_embed[tok][d] += dx[b][d][t] must not depend on scheduling.  Positions are
// sorted by token id (stable radix sort, so equal ids keep increasing (b, t) order), the dx
// tiles are transposed into a staging matrix whose rows follow the sorted order, and one block
// per distinct id adds its rows one after another onto the existing d_embed row -- the same
// sequence of fp32 additions the reference's loop performs (stories_cpu_ops.h:123-131), hence
// bit-identical to it and from run to run.
#include "common.cuh"

#include <cub/device/device_radix_sort.cuh>

namespace ane {

constexpr int EMB_THREADS = 256;

template <typename ID> __device__ __forceinline__ int load_id(const void *tokens, size_t i) {
    return (int)reinterpret_cast<const ID *>(tokens)[i];
}

// U = raw element (uint16_t / uint32_t); tile = TT tokens x DC dims, both 128 bytes wide.
template <typename U, typename ID, int TT, int DC>
__global__ void __launch_bounds__(EMB_THREADS)
embed_lookup_kernel(U *__restrict__ x, const U *__restrict__ table, const void *__restrict__ tokens, int D, int S,
                    int tiles_per_seq, int vocab, bool zero_oor, ane_cuda_status *status) {
    constexpr int PAD = sizeof(U) == 2 ? 2 : 1;  // odd row stride in 32-bit words
    __shared__ U tile[TT][DC + PAD];
    __shared__ int ids[TT];
    const int b = blockIdx.x / tiles_per_seq;
    const int t0 = (blockIdx.x % tiles_per_seq) * TT;
    const int d0 = blockIdx.y * DC;

    if (threadIdx.x < TT) {
        const int t = t0 + threadIdx.x;
        int id = -1;
        if (t < S) {
            id = load_id<ID>(tokens, (size_t)b * S + t);
            if (id < 0 || id >= vocab) {
                id = -1;
                if (blockIdx.y == 0) atomicAdd(&status->oor_ids, 1);
            }
        }
        ids[threadIdx.x] = id;
    }
    __syncthreads();
    {   // read: lanes along d
        const int dl = threadIdx.x % DC;
        for (int tl = threadIdx.x / DC; tl < TT; tl += EMB_THREADS / DC) {
            const int id = ids[tl];
            U v = 0;
            if (id >= 0 && d0 + dl < D) v = __ldg(table + (size_t)id * D + d0 + dl);
            tile[tl][dl] = v;
        }
    }
    __syncthreads();
    {   // write: lanes along t
        const int tl = threadIdx.x % TT;
        const int t = t0 + tl;
        const int id = ids[tl];
        if (t < S && (id >= 0 || zero_oor)) {
            for (int dl = threadIdx.x / TT; dl < DC; dl += EMB_THREADS / TT) {
                if (d0 + dl < D) x[((size_t)b * D + d0 + dl) * S + t] = tile[tl][dl];
            }
        }
    }
}

// ---------------------------------------------------------------- vectorised tiles
// The kernels above move one element per thread and instruction; at 2 bytes per element that is
// instruction-bound long before it is memory-bound.  The tiled forms below move 16 bytes per
// instruction on both sides.  The shared tile holds 32-bit words, tile[d][wc]: for 32-bit elements
// a word column wc is a token, for 16-bit elements it is a PAIR of adjacent tokens (low half = even
// token), so both the row side (32 bytes of one table row per thread) and the column side (16 bytes
// = 4 word columns of one channel per thread) are whole vectors.  A block covers 32 word columns
// (32 or 64 tokens) x DCW channels; row stride 36 words keeps 16-byte alignment and spreads banks.
constexpr int ET_WC = 32;           // word columns per tile
constexpr int ET_STRIDE = 36;       // words per tile row

template <int ESZ> struct EtGeom;
template <> struct EtGeom<2> { static constexpr int TOK = 64, DC = 128, CH = 16; };   // tokens, channels per tile, channels per 32-byte chunk
template <> struct EtGeom<4> { static constexpr int TOK = 32, DC = 64, CH = 8; };

// two 16-bit rows (8 channels each as uint4) -> 8 words, word j = (a[j], b[j])
__device__ __forceinline__ void interleave16(const uint4 a, const uint4 b, uint32_t (&w)[8]) {
    w[0] = __byte_perm(a.x, b.x, 0x5410); w[1] = __byte_perm(a.x, b.x, 0x7632);
    w[2] = __byte_perm(a.y, b.y, 0x5410); w[3] = __byte_perm(a.y, b.y, 0x7632);
    w[4] = __byte_perm(a.z, b.z, 0x5410); w[5] = __byte_perm(a.z, b.z, 0x7632);
    w[6] = __byte_perm(a.w, b.w, 0x5410); w[7] = __byte_perm(a.w, b.w, 0x7632);
}
// inverse of interleave16
__device__ __forceinline__ void deinterleave16(const uint32_t (&w)[8], uint4 &a, uint4 &b) {
    a.x = __byte_perm(w[0], w[1], 0x5410); b.x = __byte_perm(w[0], w[1], 0x7632);
    a.y = __byte_perm(w[2], w[3], 0x5410); b.y = __byte_perm(w[2], w[3], 0x7632);
    a.z = __byte_perm(w[4], w[5], 0x5410); b.z = __byte_perm(w[4], w[5], 0x7632);
    a.w = __byte_perm(w[6], w[7], 0x5410); b.w = __byte_perm(w[6], w[7], 0x7632);
}

// Gather.  Requirements (checked by the launcher): S % 8 == 0 (16-bit) or S % 4 == 0 (32-bit),
// D a multiple of the 32-byte chunk, 16-byte aligned x and table.
template <int ESZ, typename ID>
__global__ void __launch_bounds__(EMB_THREADS)
embed_lookup_tiled_kernel(void *__restrict__ xv, const void *__restrict__ tablev, const void *__restrict__ tokens, int D, int S,
                          int tiles_per_seq, int vocab, bool zero_oor, ane_cuda_status *status) {
    using G = EtGeom<ESZ>;
    constexpr int NCH = G::DC / G::CH;                 // 32-byte chunks per tile row: 8
    static_assert(NCH * ET_WC == EMB_THREADS, "one (word column, chunk) item per thread");
    __shared__ __align__(16) uint32_t tile[G::DC * ET_STRIDE];
    __shared__ int ids[G::TOK];
    __shared__ int any_skip;
    const int b = blockIdx.x / tiles_per_seq;
    const int t0 = (blockIdx.x % tiles_per_seq) * G::TOK;
    const int d0 = blockIdx.y * G::DC;
    const char *table = static_cast<const char *>(tablev);
    char *x = static_cast<char *>(xv);

    if (threadIdx.x == 0) any_skip = 0;
    __syncthreads();
    if (threadIdx.x < G::TOK) {
        const int t = t0 + threadIdx.x;
        int id = -1;
        if (t < S) {
            id = load_id<ID>(tokens, (size_t)b * S + t);
            if (id < 0 || id >= vocab) {
                id = -1;
                if (blockIdx.y == 0) atomicAdd(&status->oor_ids, 1);
                if (!zero_oor) any_skip = 1;
            }
        }
        ids[threadIdx.x] = id;
    }
    __syncthreads();
    {   // rows -> tile: lanes along word columns, one 32-byte chunk per warp
        const int wc = threadIdx.x % ET_WC, ch = threadIdx.x / ET_WC;
        const int d = d0 + ch * G::CH;
        if (d < D) {
            uint32_t w[8 * (ESZ == 2 ? 2 : 1)];
            if constexpr (ESZ == 2) {
                const int ia = ids[2 * wc], ib = ids[2 * wc + 1];
                uint4 a0 = make_uint4(0, 0, 0, 0), a1 = a0, b0 = a0, b1 = a0;
                if (ia >= 0) {
                    const uint4 *p = reinterpret_cast<const uint4 *>(table + ((size_t)ia * D + d) * 2);
                    a0 = __ldg(p); a1 = __ldg(p + 1);
                }
                if (ib >= 0) {
                    const uint4 *p = reinterpret_cast<const uint4 *>(table + ((size_t)ib * D + d) * 2);
                    b0 = __ldg(p); b1 = __ldg(p + 1);
                }
                uint32_t lo[8], hi[8];
                interleave16(a0, b0, lo);
                interleave16(a1, b1, hi);
#pragma unroll
                for (int j = 0; j < 8; j++) { w[j] = lo[j]; w[8 + j] = hi[j]; }
            } else {
                const int ia = ids[wc];
                uint4 a0 = make_uint4(0, 0, 0, 0), a1 = a0;
                if (ia >= 0) {
                    const uint4 *p = reinterpret_cast<const uint4 *>(table + ((size_t)ia * D + d) * 4);
                    a0 = __ldg(p); a1 = __ldg(p + 1);
                }
                w[0] = a0.x; w[1] = a0.y; w[2] = a0.z; w[3] = a0.w; w[4] = a1.x; w[5] = a1.y; w[6] = a1.z; w[7] = a1.w;
            }
#pragma unroll
            for (int j = 0; j < G::CH; j++) tile[(ch * G::CH + j) * ET_STRIDE + wc] = w[j];
        }
    }
    __syncthreads();
    // tile -> columns: 16 bytes (4 word columns) of one channel per thread
    constexpr int TPW = ESZ == 2 ? 2 : 1;              // tokens per word
    for (int item = threadIdx.x; item < G::DC * (ET_WC / 4); item += EMB_THREADS) {
        const int dl = item / (ET_WC / 4), k = item % (ET_WC / 4);
        const int t = t0 + k * 4 * TPW;
        if (d0 + dl >= D || t >= S) continue;
        const uint4 v = *reinterpret_cast<const uint4 *>(&tile[dl * ET_STRIDE + 4 * k]);
        char *dst = x + (((size_t)b * D + d0 + dl) * S + t) * ESZ;
        if (!any_skip) {
            __stcs(reinterpret_cast<uint4 *>(dst), v);
        } else {        // some token of this tile keeps its stale column: element-wise stores
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4 * TPW; q++) {
                if (ids[k * 4 * TPW + q] < 0) continue;
                if constexpr (ESZ == 2) reinterpret_cast<uint16_t *>(dst)[q] = (uint16_t)(w[q / 2] >> (16 * (q & 1)));
                else reinterpret_cast<uint32_t *>(dst)[q] = w[q];
            }
        }
    }
}

// ---------------------------------------------------------------- scatter-add
template <typename ID>
__global__ void eb_prepare_kernel(int *__restrict__ keys, int *__restrict__ vals, const void *__restrict__ tokens,
                                  int n, int vocab, ane_cuda_status *status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int id = load_id<ID>(tokens, i);
    if (id < 0 || id >= vocab) { id = vocab; atomicAdd(&status->oor_ids, 1); }   // sorts behind every valid id
    keys[i] = id;
    vals[i] = i;
}

__global__ void eb_inverse_kernel(int *__restrict__ rank_of_pos, const int *__restrict__ sorted_pos, int n) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < n) rank_of_pos[sorted_pos[r]] = r;
}

// dx [B][D][S] tile -> stage[rank(b,t)][d]  (raw elements)
template <typename U, int TT, int DC>
__global__ void __launch_bounds__(EMB_THREADS)
eb_stage_kernel(U *__restrict__ stage, const U *__restrict__ dx, const int *__restrict__ rank_of_pos, int D, int S,
                int tiles_per_seq) {
    constexpr int PAD = sizeof(U) == 2 ? 2 : 1;
    __shared__ U tile[TT][DC + PAD];
    __shared__ int ranks[TT];
    const int b = blockIdx.x / tiles_per_seq;
    const int t0 = (blockIdx.x % tiles_per_seq) * TT;
    const int d0 = blockIdx.y * DC;
    if (threadIdx.x < TT) {
        const int t = t0 + threadIdx.x;
        ranks[threadIdx.x] = t < S ? rank_of_pos[(size_t)b * S + t] : -1;
    }
    {   // read: lanes along t
        const int tl = threadIdx.x % TT;
        const int t = t0 + tl;
        for (int dl = threadIdx.x / TT; dl < DC; dl += EMB_THREADS / TT) {
            U v = 0;
            if (t < S && d0 + dl < D) v = __ldcs(dx + ((size_t)b * D + d0 + dl) * S + t);
            tile[tl][dl] = v;
        }
    }
    __syncthreads();
    {   // write: lanes along d
        const int dl = threadIdx.x % DC;
        for (int tl = threadIdx.x / DC; tl < TT; tl += EMB_THREADS / DC) {
            const int r = ranks[tl];
            if (r >= 0 && d0 + dl < D) stage[(size_t)r * D + d0 + dl] = tile[tl][dl];
        }
    }
}

// One block per sorted rank; the first rank of each id walks its run and adds onto d_embed.
template <typename T>
__global__ void __launch_bounds__(128)
eb_reduce_kernel(float *__restrict__ d_embed, const T *__restrict__ stage, const int *__restrict__ keys, int n, int D,
                 int vocab) {
    const int r = blockIdx.x;
    const int key = keys[r];
    if (key >= vocab) return;                       // out-of-range ids are skipped (stories_cpu_ops.h:126)
    if (r > 0 && keys[r - 1] == key) return;        // not the first of its run
    int end = r + 1;
    while (end < n && keys[end] == key) end++;
    for (int d = threadIdx.x; d < D; d += 128) {
        float acc = d_embed[(size_t)key * D + d];
        for (int q = r; q < end; q++) acc += Elt<T>::to_f(stage[(size_t)q * D + d]);
        d_embed[(size_t)key * D + d] = acc;
    }
}

// Gather, row-walking form (the mirror image of eb_stage_rows_kernel below): a block takes 32 tokens
// (16 word columns) x up to 512 channels; a WARP owns a word column and walks its table row(s) with
// consecutive lanes on consecutive channels (one sequential 1-2 KB burst per row), the column side
// writes 64-byte segments of x.
constexpr int ER_WC = 16, ER_DC = 512, ER_STRIDE = 17, ER_THREADS = 32 * ER_WC;

template <int ESZ, typename ID>
__global__ void __launch_bounds__(ER_THREADS)
embed_lookup_rows_kernel(void *__restrict__ xv, const void *__restrict__ tablev, const void *__restrict__ tokens, int D, int S,
                         int tiles_per_seq, int vocab, bool zero_oor, ane_cuda_status *status) {
    constexpr int TPW = ESZ == 2 ? 2 : 1;
    constexpr int TOK = ER_WC * TPW;
    __shared__ uint32_t tile[ER_DC * ER_STRIDE];
    __shared__ int ids[TOK];
    __shared__ int any_skip;
    const int b = blockIdx.x / tiles_per_seq;
    const int t0 = (blockIdx.x % tiles_per_seq) * TOK;
    const int d0 = blockIdx.y * ER_DC;
    const int dcount = D - d0 < ER_DC ? D - d0 : ER_DC;
    const char *table = static_cast<const char *>(tablev);
    char *x = static_cast<char *>(xv);

    if (threadIdx.x == 0) any_skip = 0;
    __syncthreads();
    if (threadIdx.x < TOK) {
        const int t = t0 + threadIdx.x;
        int id = -1;
        if (t < S) {
            id = load_id<ID>(tokens, (size_t)b * S + t);
            if (id < 0 || id >= vocab) {
                id = -1;
                if (blockIdx.y == 0) atomicAdd(&status->oor_ids, 1);
                if (!zero_oor) any_skip = 1;
            }
        }
        ids[threadIdx.x] = id;
    }
    __syncthreads();
    {   // rows -> tile: four channels per lane and step
        const int wc = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int nquad = dcount >> 2;
        if constexpr (ESZ == 2) {
            const int ia = ids[2 * wc], ib = ids[2 * wc + 1];
            const uint2 *ra = reinterpret_cast<const uint2 *>(table + ((size_t)(ia < 0 ? 0 : ia) * D + d0) * 2);
            const uint2 *rb = reinterpret_cast<const uint2 *>(table + ((size_t)(ib < 0 ? 0 : ib) * D + d0) * 2);
#pragma unroll 4
            for (int cq = lane; cq < nquad; cq += 32) {
                uint2 a = make_uint2(0, 0), c = make_uint2(0, 0);
                if (ia >= 0) a = __ldg(ra + cq);
                if (ib >= 0) c = __ldg(rb + cq);
                uint32_t *col = &tile[(4 * cq) * ER_STRIDE + wc];
                col[0] = __byte_perm(a.x, c.x, 0x5410);
                col[ER_STRIDE] = __byte_perm(a.x, c.x, 0x7632);
                col[2 * ER_STRIDE] = __byte_perm(a.y, c.y, 0x5410);
                col[3 * ER_STRIDE] = __byte_perm(a.y, c.y, 0x7632);
            }
        } else {
            const int ia = ids[wc];
            const uint4 *ra = reinterpret_cast<const uint4 *>(table + ((size_t)(ia < 0 ? 0 : ia) * D + d0) * 4);
#pragma unroll 4
            for (int cq = lane; cq < nquad; cq += 32) {
                uint4 a = make_uint4(0, 0, 0, 0);
                if (ia >= 0) a = __ldg(ra + cq);
                uint32_t *col = &tile[(4 * cq) * ER_STRIDE + wc];
                col[0] = a.x; col[ER_STRIDE] = a.y; col[2 * ER_STRIDE] = a.z; col[3 * ER_STRIDE] = a.w;
            }
        }
    }
    __syncthreads();
    constexpr int VPR = ER_WC / 4;                       // 16-byte vectors per tile row
    for (int item = threadIdx.x; item < dcount * VPR; item += ER_THREADS) {
        const int dl = item / VPR, k = item % VPR;
        const int t = t0 + k * 4 * TPW;
        if (t >= S) continue;
        const uint32_t *row = &tile[dl * ER_STRIDE + 4 * k];
        const uint32_t w[4] = {row[0], row[1], row[2], row[3]};
        char *dst = x + (((size_t)b * D + d0 + dl) * S + t) * ESZ;
        if (!any_skip) {
            __stcs(reinterpret_cast<uint4 *>(dst), make_uint4(w[0], w[1], w[2], w[3]));
        } else {        // some token of this tile keeps its stale column: element-wise stores
#pragma unroll
            for (int q = 0; q < 4 * TPW; q++) {
                if (ids[k * 4 * TPW + q] < 0) continue;
                if constexpr (ESZ == 2) reinterpret_cast<uint16_t *>(dst)[q] = (uint16_t)(w[q / 2] >> (16 * (q & 1)));
                else reinterpret_cast<uint32_t *>(dst)[q] = w[q];
            }
        }
    }
}

// ---------------------------------------------------------------- vectorised scatter-add
// Staging kernel destinations:
//   dest >= 0       row `dest` (= the position b*S + t itself) of the staging matrix: the id occurs more
//                   than once and its rows are added in position order by eb_reduce_runs_kernel;
//   EB_SKIP         out-of-range id, dropped (stories_cpu_ops.h:126);
//   otherwise       -(id + 2): the id occurs exactly once, so its column is added straight onto
//                   d_embed[id] -- a single addition has no order to preserve, and the staging
//                   round trip (one write and one read of the column) is saved.
// Only the reduction of repeated ids needs the positions sorted by id; that sort depends on the
// tokens alone and runs on a side stream while the staging kernel moves the data.
constexpr int EB_SKIP = -1;

// sort keys: out-of-range ids sort behind every valid id
template <typename ID>
__global__ void eb_keys_kernel(int *__restrict__ keys, int *__restrict__ vals, const void *__restrict__ tokens, int n, int vocab) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int id = load_id<ID>(tokens, i);
    if (id < 0 || id >= vocab) id = vocab;
    keys[i] = id;
    vals[i] = i;
}

// starts of runs longer than one go to a work list (its order does not matter: runs are independent)
__global__ void eb_runs_kernel(int *__restrict__ run_start, int *__restrict__ run_count, const int *__restrict__ keys, int n, int vocab) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n) return;
    const int key = keys[r];
    if (key >= vocab) return;
    const bool first = r == 0 || keys[r - 1] != key;
    const bool last = r == n - 1 || keys[r + 1] != key;
    if (first && !last) run_start[atomicAdd(run_count, 1)] = r;
}

template <typename T> __device__ __forceinline__ float raw16_to_f(uint32_t h);
template <> __device__ __forceinline__ float raw16_to_f<__nv_bfloat16>(uint32_t h) { return __uint_as_float(h << 16); }
template <> __device__ __forceinline__ float raw16_to_f<__half>(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

// Staging kernel.  Random 64-byte read-modify-writes of d_embed (every lane of a warp on a different
// row, what a 64-token x 128-channel tile leads to) ran at a tenth of the HBM rate: each touches its own
// DRAM page.  Here a block takes 32 tokens (16 word columns) x up to 512 channels, and a WARP owns a
// word column: it walks its half of the d_embed (or staging) row with consecutive lanes on consecutive
// channels, so every row piece is one sequential 1-2 KB burst.  The column side reads 64-byte segments
// of dx (32-byte segments cost a 64-byte DRAM fetch each).

// occurrences of every id (count must be zero on entry); out-of-range ids are reported, not counted
template <typename ID>
__global__ void eb_count_kernel(int *__restrict__ count, const void *__restrict__ tokens, int n, int vocab, ane_cuda_status *status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int id = load_id<ID>(tokens, i);
    if (id < 0 || id >= vocab) atomicAdd(&status->oor_ids, 1);
    else atomicAdd(&count[id], 1);
}

// Destination of a position, from the occurrence counts alone (no sort needed): an id that occurs once
// goes straight to d_embed, any other to the staging row of its own position.
template <typename ID>
__device__ __forceinline__ int eb_dest(const void *tokens, const int *count, size_t pos, int vocab) {
    const int id = load_id<ID>(tokens, pos);
    if (id < 0 || id >= vocab) return EB_SKIP;
    return count[id] == 1 ? -(id + 2) : (int)pos;
}

template <typename T, int ESZ, typename ID>
__global__ void __launch_bounds__(ER_THREADS)
eb_stage_rows_kernel(void *__restrict__ stagev, float *__restrict__ d_embed, const void *__restrict__ dxv,
                     const void *__restrict__ tokens, const int *__restrict__ count, int vocab, int D, int S, int tiles_per_seq,
                     const int *__restrict__ seg_start, const int *__restrict__ arr_of_pos, int *__restrict__ seg_pos) {
    constexpr int TPW = ESZ == 2 ? 2 : 1;
    constexpr int TOK = ER_WC * TPW;
    __shared__ uint32_t tile[ER_DC * ER_STRIDE];
    __shared__ int dst[TOK];
    const int b = blockIdx.x / tiles_per_seq;
    const int t0 = (blockIdx.x % tiles_per_seq) * TOK;
    const int d0 = blockIdx.y * ER_DC;
    const int dcount = D - d0 < ER_DC ? D - d0 : ER_DC;
    const char *dx = static_cast<const char *>(dxv);

    if (threadIdx.x < TOK) {
        const int t = t0 + threadIdx.x;
        const int dsel = t < S ? eb_dest<ID>(tokens, count, (size_t)b * S + t, vocab) : EB_SKIP;
        dst[threadIdx.x] = dsel;
        // the sort-free form: a repeated position is filed in its id's segment, at its arrival number
        if (seg_pos && dsel >= 0 && blockIdx.y == 0) seg_pos[seg_start[load_id<ID>(tokens, (size_t)dsel)] + arr_of_pos[dsel]] = dsel;
    }
    constexpr int VPR = ER_WC / 4;                       // 16-byte vectors per tile row
    for (int item = threadIdx.x; item < dcount * VPR; item += ER_THREADS) {
        const int dl = item / VPR, k = item % VPR;
        const int t = t0 + k * 4 * TPW;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t < S) v = __ldcs(reinterpret_cast<const uint4 *>(dx + (((size_t)b * D + d0 + dl) * S + t) * ESZ));
        uint32_t *row = &tile[dl * ER_STRIDE + 4 * k];
        row[0] = v.x; row[1] = v.y; row[2] = v.z; row[3] = v.w;
    }
    __syncthreads();
    const int wc = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int npair = dcount >> 1;                       // channel pairs
#pragma unroll
    for (int q = 0; q < TPW; q++) {
        const int dsel = dst[wc * TPW + q];
        if (dsel == EB_SKIP) continue;
        // value pair (channels 2cp, 2cp+1) of this token
        auto fetch = [&](int cp, float &f0, float &f1, uint32_t &raw) {
            const uint32_t w0 = tile[(2 * cp) * ER_STRIDE + wc], w1 = tile[(2 * cp + 1) * ER_STRIDE + wc];
            if constexpr (ESZ == 2) {
                raw = __byte_perm(w0, w1, q == 0 ? 0x5410 : 0x7632);
                f0 = raw16_to_f<T>(raw & 0xffffu);
                f1 = raw16_to_f<T>(raw >> 16);
            } else {
                raw = 0;
                f0 = __uint_as_float(w0);
                f1 = __uint_as_float(w1);
            }
        };
        if (dsel >= 0) {
            char *srow = static_cast<char *>(stagev) + ((size_t)dsel * D + d0) * ESZ;
            for (int cp = lane; cp < npair; cp += 32) {
                float f0, f1;
                uint32_t raw;
                fetch(cp, f0, f1, raw);
                if constexpr (ESZ == 2) reinterpret_cast<uint32_t *>(srow)[cp] = raw;
                else reinterpret_cast<float2 *>(srow)[cp] = make_float2(f0, f1);
            }
        } else {
            float2 *erow = reinterpret_cast<float2 *>(d_embed + (size_t)(-(dsel + 2)) * D + d0);
            constexpr int UN = 8;
            for (int cb = lane; cb < npair; cb += 32 * UN) {
                float2 cur[UN];
#pragma unroll
                for (int u = 0; u < UN; u++)
                    if (cb + u * 32 < npair) cur[u] = erow[cb + u * 32];
#pragma unroll
                for (int u = 0; u < UN; u++) {
                    const int cp = cb + u * 32;
                    if (cp < npair) {
                        float f0, f1;
                        uint32_t raw;
                        fetch(cp, f0, f1, raw);
                        erow[cp] = make_float2(cur[u].x + f0, cur[u].y + f1);
                    }
                }
            }
        }
    }
}

// Runs of equal ids (length >= 2): a WARP per run adds the staging rows in sorted (= position) order
// onto the d_embed row, four channels per lane and step.  With one warp per run all runs are in flight
// at once, which hides the chain of dependent loads (keys, positions, rows) each of them is.
constexpr int RR_THREADS = 256, RR_J = 8;
template <typename T, int ESZ>
__device__ __forceinline__ void rr_add(float4 &acc, const uint4 raw) {
    if constexpr (ESZ == 2) {
        acc.x += raw16_to_f<T>(raw.x & 0xffffu); acc.y += raw16_to_f<T>(raw.x >> 16);
        acc.z += raw16_to_f<T>(raw.y & 0xffffu); acc.w += raw16_to_f<T>(raw.y >> 16);
    } else {
        acc.x += __uint_as_float(raw.x); acc.y += __uint_as_float(raw.y);
        acc.z += __uint_as_float(raw.z); acc.w += __uint_as_float(raw.w);
    }
}
template <int ESZ>
__device__ __forceinline__ uint4 rr_load(const char *src) {
    if constexpr (ESZ == 2) {
        const uint2 v = *reinterpret_cast<const uint2 *>(src);
        return make_uint4(v.x, v.y, 0, 0);
    } else {
        return *reinterpret_cast<const uint4 *>(src);
    }
}

template <typename T, int ESZ>
__global__ void __launch_bounds__(RR_THREADS)
eb_reduce_runs_kernel(float *__restrict__ d_embed, const void *__restrict__ stagev, const int *__restrict__ keys,
                      const int *__restrict__ sorted_pos, const int *__restrict__ run_start, const int *__restrict__ run_count,
                      int n, int D) {
    const char *stage = static_cast<const char *>(stagev);
    const int lane = threadIdx.x & 31;
    const int wi = blockIdx.x * (RR_THREADS / 32) + (threadIdx.x >> 5);
    if (wi >= *run_count) return;
    const int r = run_start[wi];
    const int key = keys[r];
    float *erow = d_embed + (size_t)key * D;
    for (int d0 = 0; d0 < D; d0 += 128 * RR_J) {
        float4 acc[RR_J];
#pragma unroll
        for (int j = 0; j < RR_J; j++) {
            const int d = d0 + (j * 32 + lane) * 4;
            if (d < D) acc[j] = *reinterpret_cast<const float4 *>(erow + d);
        }
        for (int q0 = r;; q0 += 32) {                    // 32 positions of the run per round
            const int idx = q0 + lane;
            const bool same = idx < n && keys[idx] == key;
            const unsigned m = __ballot_sync(0xffffffffu, same);
            const int cnt = m == 0xffffffffu ? 32 : __ffs(~m) - 1;
            const int mypos = same ? sorted_pos[idx] : 0;
            for (int u = 0; u < cnt; u += 2) {           // two rows (16 loads) in flight; added in order
                const size_t row0 = (size_t)__shfl_sync(0xffffffffu, mypos, u) * D;
                const size_t row1 = (size_t)__shfl_sync(0xffffffffu, mypos, (u + 1) & 31) * D;
                const bool two = u + 1 < cnt;
                uint4 v0[RR_J], v1[RR_J];
#pragma unroll
                for (int j = 0; j < RR_J; j++) {
                    const int d = d0 + (j * 32 + lane) * 4;
                    if (d < D) {
                        v0[j] = rr_load<ESZ>(stage + (row0 + d) * ESZ);
                        if (two) v1[j] = rr_load<ESZ>(stage + (row1 + d) * ESZ);
                    }
                }
#pragma unroll
                for (int j = 0; j < RR_J; j++) {
                    const int d = d0 + (j * 32 + lane) * 4;
                    if (d < D) {
                        rr_add<T, ESZ>(acc[j], v0[j]);
                        if (two) rr_add<T, ESZ>(acc[j], v1[j]);
                    }
                }
            }
            if (cnt < 32) break;
        }
#pragma unroll
        for (int j = 0; j < RR_J; j++) {
            const int d = d0 + (j * 32 + lane) * 4;
            if (d < D) *reinterpret_cast<float4 *>(erow + d) = acc[j];
        }
    }
}

// ---------------------------------------------------------------- scatter-add without a sort
// The sort above exists only to put the positions of a repeated id into increasing order.  Repeated ids are few and
// their runs short (uniform ids over a 152 k vocabulary: 10 k runs of 2.2 positions on average in 65 k tokens), so
// here the order is made where it is needed instead:
//   eb_count_arrival   count[id]++ gives every position its arrival number within its id (any order);
//   eb_segments        every id that occurs twice or more gets a segment of count[id] slots in a position list and an
//                      entry in the list of runs (one atomic per block, not per id);
//   eb_stage_rows      the staging kernel above; on its way it files each repeated position in its id's segment;
//   eb_reduce_segments a warp per (run, 256-channel piece) sorts the run's positions -- up to 32 in registers, up to 256 by
//                      counting ranks, longer runs by walking the token array in order -- and adds the staging rows onto
//                      the d_embed row in increasing position order: the reference's additions in the reference's order.
constexpr int EB_INLINE_MAX = 32;      // positions of a run sorted in registers
constexpr int EB_RANK_MAX = 256;       // longer runs: ranked by counting up to here, found by a walk over the tokens beyond
struct EbLists {
    int *count;        // [vocab]  occurrences per id
    int *seg_start;    // [vocab]  first slot of an id's segment (ids with count >= 2)
    int *arr_of_pos;   // [n]      arrival number of a position within its id
    int *seg_pos;      // [n]      positions, grouped by id, in arrival order
    int4 *run_info;    // [n / 2]  (id, count, first slot, 0) of every id with count >= 2
    int *cursor;       // [0] slots handed out, [1] runs
};

template <typename ID>
__global__ void eb_count_arrival_kernel(EbLists L, const void *__restrict__ tokens, int n, int vocab, ane_cuda_status *status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int id = load_id<ID>(tokens, i);
    if (id < 0 || id >= vocab) atomicAdd(&status->oor_ids, 1);
    else L.arr_of_pos[i] = atomicAdd(&L.count[id], 1);
}

constexpr int SEG_THREADS = 1024;
__global__ void __launch_bounds__(SEG_THREADS) eb_segments_kernel(EbLists L, int vocab) {
    __shared__ int wsum[2][SEG_THREADS / 32];
    __shared__ int base[2];
    const int id = blockIdx.x * SEG_THREADS + threadIdx.x;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int c = id < vocab ? L.count[id] : 0;
    const int slots = c >= 2 ? c : 0, isrun = c >= 2 ? 1 : 0;
    int ps = slots, pr = isrun;                          // inclusive scans over the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, ps, o), r = __shfl_up_sync(0xffffffffu, pr, o);
        if (lane >= o) { ps += a; pr += r; }
    }
    if (lane == 31) { wsum[0][w] = ps; wsum[1][w] = pr; }
    __syncthreads();
    if (w == 0) {
        int a = wsum[0][lane], r = wsum[1][lane];        // SEG_THREADS / 32 == 32 warps
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int a2 = __shfl_up_sync(0xffffffffu, a, o), r2 = __shfl_up_sync(0xffffffffu, r, o);
            if (lane >= o) { a += a2; r += r2; }
        }
        if (lane == 31) { base[0] = a ? atomicAdd(&L.cursor[0], a) : 0; base[1] = r ? atomicAdd(&L.cursor[1], r) : 0; }
        wsum[0][lane] = a - wsum[0][lane];               // exclusive offsets of the warps
        wsum[1][lane] = r - wsum[1][lane];
    }
    __syncthreads();
    if (isrun) {
        L.seg_start[id] = base[0] + wsum[0][w] + ps - slots;
        L.run_info[base[1] + wsum[1][w] + pr - 1] = make_int4(id, c, base[0] + wsum[0][w] + ps - slots, 0);
    }
}

// cnt (<= 32) staging row pieces, lane u holding the position of the u-th, added onto acc in that order
template <typename T, int ESZ, int NJ>
__device__ __forceinline__ void eb_add_rows_in_order(float4 (&acc)[NJ], const char *stage, int D, int d0, int dcount, int lane,
                                                     int mypos, int cnt) {
    for (int u = 0; u < cnt; u += 2) {                   // two rows in flight; added in order
        const size_t row0 = (size_t)__shfl_sync(0xffffffffu, mypos, u) * D;
        const size_t row1 = (size_t)__shfl_sync(0xffffffffu, mypos, (u + 1) & 31) * D;
        const bool two = u + 1 < cnt;
        uint4 v0[NJ], v1[NJ];
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            const int d = (j * 32 + lane) * 4;
            if (d < dcount) {
                v0[j] = rr_load<ESZ>(stage + (row0 + d0 + d) * ESZ);
                if (two) v1[j] = rr_load<ESZ>(stage + (row1 + d0 + d) * ESZ);
            }
        }
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            const int d = (j * 32 + lane) * 4;
            if (d < dcount) {
                rr_add<T, ESZ>(acc[j], v0[j]);
                if (two) rr_add<T, ESZ>(acc[j], v1[j]);
            }
        }
    }
}

constexpr int RS_THREADS = 256, RS_J = 2, RS_CH = 128 * RS_J;     // a warp item covers RS_CH channels of a run
#ifndef ANE_RS_MINB
#define ANE_RS_MINB 4
#endif
template <typename T, int ESZ, typename ID>
__global__ void __launch_bounds__(RS_THREADS, ANE_RS_MINB)
eb_reduce_segments_kernel(float *__restrict__ d_embed, const void *__restrict__ stagev, const void *__restrict__ tokens, EbLists L,
                          int n, int D) {
    __shared__ int sorted[RS_THREADS / 32][EB_RANK_MAX];
    const char *stage = static_cast<const char *>(stagev);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int nruns = L.cursor[1];
    const int pieces = (D + RS_CH - 1) / RS_CH;
    const long long nitems = (long long)nruns * pieces;
    for (long long item = (long long)blockIdx.x * (RS_THREADS / 32) + w; item < nitems; item += (long long)gridDim.x * (RS_THREADS / 32)) {
        const int4 info = L.run_info[item / pieces];
        const int key = info.x, cnt = info.y, s = info.z;
        const int d0 = (int)(item % pieces) * RS_CH;
        const int dcount = D - d0 < RS_CH ? D - d0 : RS_CH;
        float *erow = d_embed + (size_t)key * D + d0;
        float4 acc[RS_J];
#pragma unroll
        for (int j = 0; j < RS_J; j++) {                 // the d_embed row piece: in flight while the positions are sorted
            const int d = (j * 32 + lane) * 4;
            if (d < dcount) acc[j] = *reinterpret_cast<const float4 *>(erow + d);
        }
        if (cnt <= EB_INLINE_MAX) {
            const int mine = lane < cnt ? L.seg_pos[s + lane] : 0x7fffffff;
            int rank = 0;
            for (int j = 0; j < cnt; j++) rank += __shfl_sync(0xffffffffu, mine, j) < mine;
            if (lane < cnt) sorted[w][rank] = mine;
            __syncwarp();
            const int mypos = lane < cnt ? sorted[w][lane] : 0;
            __syncwarp();
            eb_add_rows_in_order<T, ESZ, RS_J>(acc, stage, D, d0, dcount, lane, mypos, cnt);
        } else if (cnt <= EB_RANK_MAX) {
            for (int i = lane; i < cnt; i += 32) {
                const int p = L.seg_pos[s + i];
                int rank = 0;
                for (int j = 0; j < cnt; j++) rank += L.seg_pos[s + j] < p;
                sorted[w][rank] = p;
            }
            __syncwarp();
            for (int q0 = 0; q0 < cnt; q0 += 32) {
                const int c = cnt - q0 < 32 ? cnt - q0 : 32;
                const int mypos = lane < c ? sorted[w][q0 + lane] : 0;
                eb_add_rows_in_order<T, ESZ, RS_J>(acc, stage, D, d0, dcount, lane, mypos, c);
            }
            __syncwarp();
        } else {
            for (int q0 = 0; q0 < n; q0 += 32) {
                const int idx = q0 + lane;
                const bool same = idx < n && load_id<ID>(tokens, idx) == key;
                const unsigned m = __ballot_sync(0xffffffffu, same);
                if (m == 0) continue;
                const int c = __popc(m);
                const int mypos = lane < c ? q0 + (int)__fns(m, 0, lane + 1) : 0;
                eb_add_rows_in_order<T, ESZ, RS_J>(acc, stage, D, d0, dcount, lane, mypos, c);
            }
        }
#pragma unroll
        for (int j = 0; j < RS_J; j++) {
            const int d = (j * 32 + lane) * 4;
            if (d < dcount) *reinterpret_cast<float4 *>(erow + d) = acc[j];
        }
    }
}

// Side stream for the sort (created on first use, destroyed at shutdown).
struct EmbedSide { cudaStream_t stream = nullptr; cudaEvent_t fork = nullptr, join = nullptr; bool ok = false; };
static EmbedSide g_side;
static EmbedSide *embed_side() {
    if (g_side.ok) return &g_side;
    int lo = 0, hi = 0;                                  // the short sort kernels must not queue behind the data movement
    cudaDeviceGetStreamPriorityRange(&lo, &hi);
    if (cudaStreamCreateWithPriority(&g_side.stream, cudaStreamNonBlocking, hi) != cudaSuccess ||
        cudaEventCreateWithFlags(&g_side.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&g_side.join, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    g_side.ok = true;
    return &g_side;
}
void embed_side_release() {
    if (g_side.stream) cudaStreamDestroy(g_side.stream);
    if (g_side.fork) cudaEventDestroy(g_side.fork);
    if (g_side.join) cudaEventDestroy(g_side.join);
    g_side = EmbedSide();
}

static int sort_bits(int vocab) {
    int bits = 1;
    while ((1ll << bits) <= (long long)vocab) bits++;   // keys go up to `vocab` (the out-of-range sentinel)
    return bits;
}

}  // namespace ane

using namespace ane;

extern "C" {

int ane_cuda_embed_lookup_dev(void *stream, ane_dtype dtype, ane_idtype idtype, int B, int D, int S, void *x,
                              const void *table, const void *tokens, int vocab, unsigned flags) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(x && table && tokens, "%s: null pointer", __func__);
    ANE_REQUIRE(dtype_ok(dtype), "%s: bad dtype", __func__);
    ANE_REQUIRE(idtype == ANE_ID_U16 || idtype == ANE_ID_I32, "%s: bad id type", __func__);
    ANE_REQUIRE(B >= 1 && D >= 1 && S >= 1 && vocab >= 1, "%s: bad shape B=%d D=%d S=%d vocab=%d", __func__, B, D, S, vocab);
    ANE_REQUIRE(flags == ANE_OOR_SKIP || flags == ANE_OOR_ZERO, "%s: bad flags %u", __func__, flags);
    ANE_CHECK_EXTENT(x, (size_t)B * D * S * dtype_size(dtype)); ANE_CHECK_EXTENT(table, (size_t)vocab * D * dtype_size(dtype));
    ANE_CHECK_EXTENT(tokens, (size_t)B * S * (idtype == ANE_ID_U16 ? 2 : 4));
    cudaStream_t st = (cudaStream_t)stream;
    const bool zero = flags == ANE_OOR_ZERO;
    ane_cuda_status *status = ctx().status;
    const size_t esz = dtype_size(dtype);
    const bool tiled = tuning("embed_tiled", 1) && aligned16(x) && aligned16(table) && S % (16 / (int)esz) == 0 &&
                       D % (32 / (int)esz) == 0;
    if (tiled && tuning("embed_rows", 1) && D % 4 == 0) {
        const int TOKr = ER_WC * (esz == 2 ? 2 : 1);
        const int tps = (S + TOKr - 1) / TOKr;
        dim3 grid((unsigned)(B * tps), (unsigned)((D + ER_DC - 1) / ER_DC));
        if (esz == 2) {
            if (idtype == ANE_ID_U16) embed_lookup_rows_kernel<2, uint16_t><<<grid, ER_THREADS, 0, st>>>(x, table, tokens, D, S, tps, vocab, zero, status);
            else embed_lookup_rows_kernel<2, int32_t><<<grid, ER_THREADS, 0, st>>>(x, table, tokens, D, S, tps, vocab, zero, status);
        } else {
            if (idtype == ANE_ID_U16) embed_lookup_rows_kernel<4, uint16_t><<<grid, ER_THREADS, 0, st>>>(x, table, tokens, D, S, tps, vocab, zero, status);
            else embed_lookup_rows_kernel<4, int32_t><<<grid, ER_THREADS, 0, st>>>(x, table, tokens, D, S, tps, vocab, zero, status);
        }
    } else if (tiled && esz == 2) {
        using G = EtGeom<2>;
        const int tps = (S + G::TOK - 1) / G::TOK;
        dim3 grid((unsigned)(B * tps), (unsigned)((D + G::DC - 1) / G::DC));
        if (idtype == ANE_ID_U16) embed_lookup_tiled_kernel<2, uint16_t><<<grid, EMB_THREADS, 0, st>>>(x, table, tokens, D, S, tps, vocab, zero, status);
        else embed_lookup_tiled_kernel<2, int32_t><<<grid, EMB_THREADS, 0, st>>>(x, table, tokens, D, S, tps, vocab, zero, status);
    } else if (tiled) {
        using G = EtGeom<4>;
        const int tps = (S + G::TOK - 1) / G::TOK;
        dim3 grid((unsigned)(B * tps), (unsigned)((D + G::DC - 1) / G::DC));
        if (idtype == ANE_ID_U16) embed_lookup_tiled_kernel<4, uint16_t><<<grid, EMB_THREADS, 0, st>>>(x, table, tokens, D, S, tps, vocab, zero, status);
        else embed_lookup_tiled_kernel<4, int32_t><<<grid, EMB_THREADS, 0, st>>>(x, table, tokens, D, S, tps, vocab, zero, status);
    } else if (dtype == ANE_F32) {
        constexpr int TT = 32, DC = 32;
        const int tps = (S + TT - 1) / TT;
        dim3 grid((unsigned)(B * tps), (unsigned)((D + DC - 1) / DC));
        if (idtype == ANE_ID_U16)
            embed_lookup_kernel<uint32_t, uint16_t, TT, DC><<<grid, EMB_THREADS, 0, st>>>((uint32_t *)x, (const uint32_t *)table, tokens, D, S, tps, vocab, zero, status);
        else
            embed_lookup_kernel<uint32_t, int32_t, TT, DC><<<grid, EMB_THREADS, 0, st>>>((uint32_t *)x, (const uint32_t *)table, tokens, D, S, tps, vocab, zero, status);
    } else {
        constexpr int TT = 64, DC = 64;
        const int tps = (S + TT - 1) / TT;
        dim3 grid((unsigned)(B * tps), (unsigned)((D + DC - 1) / DC));
        if (idtype == ANE_ID_U16)
            embed_lookup_kernel<uint16_t, uint16_t, TT, DC><<<grid, EMB_THREADS, 0, st>>>((uint16_t *)x, (const uint16_t *)table, tokens, D, S, tps, vocab, zero, status);
        else
            embed_lookup_kernel<uint16_t, int32_t, TT, DC><<<grid, EMB_THREADS, 0, st>>>((uint16_t *)x, (const uint16_t *)table, tokens, D, S, tps, vocab, zero, status);
    }
    ANE_LAUNCH_OK(1);
    return ANE_CUDA_OK;
}

int ane_cuda_embed_backward_dev(void *stream, ane_dtype dtype, ane_idtype idtype, int B, int D, int S, float *d_embed,
                                const void *dx, const void *tokens, int vocab) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(d_embed && dx && tokens, "%s: null pointer", __func__);
    ANE_REQUIRE(dtype_ok(dtype), "%s: bad dtype", __func__);
    ANE_REQUIRE(idtype == ANE_ID_U16 || idtype == ANE_ID_I32, "%s: bad id type", __func__);
    ANE_REQUIRE(B >= 1 && D >= 1 && S >= 1 && vocab >= 1, "%s: bad shape B=%d D=%d S=%d vocab=%d", __func__, B, D, S, vocab);
    ANE_REQUIRE((long long)B * S < 0x7fffffffLL, "%s: too many tokens", __func__);
    ANE_CHECK_EXTENT(d_embed, (size_t)vocab * D * 4); ANE_CHECK_EXTENT(dx, (size_t)B * D * S * dtype_size(dtype));
    ANE_CHECK_EXTENT(tokens, (size_t)B * S * (idtype == ANE_ID_U16 ? 2 : 4));
    cudaStream_t st = (cudaStream_t)stream;
    const int n = B * S;
    const size_t esz = dtype_size(dtype);
    const bool u16 = idtype == ANE_ID_U16;

    const bool tiled = tuning("embed_tiled", 1) && aligned16(dx) && aligned16(d_embed) && S % (16 / (int)esz) == 0 && D % 4 == 0;
    const size_t ints = round_up((size_t)n * sizeof(int), 256);
    const int pb = (n + 255) / 256;
    if (tiled && !tuning("embed_sort", 0)) {
        // no sort: arrival numbers -> segments and run list -> staging kernel (files the repeated positions) -> ordered adds per run
        const size_t o_cursor = 0;                                                           // 64 ints
        const size_t o_count = 256;
        const size_t o_zero_end = o_count + round_up((size_t)vocab * sizeof(int), 256);      // everything up to here starts at zero
        const size_t o_seg = o_zero_end;
        const size_t o_arr = o_seg + round_up((size_t)vocab * sizeof(int), 256);
        const size_t o_pos = o_arr + ints;
        const size_t o_run = o_pos + ints;
        const size_t o_stage2 = o_run + round_up(((size_t)n / 2 + 1) * sizeof(int4), 256);
        const size_t total2 = o_stage2 + round_up((size_t)n * D * esz, 256);
        char *ws2 = static_cast<char *>(workspace(total2));
        if (!ws2) return fail(ANE_CUDA_ERR_NOMEM, "%s: no scratch (%zu bytes)", __func__, total2);
        EbLists L;
        L.cursor = (int *)(ws2 + o_cursor);
        L.count = (int *)(ws2 + o_count);
        L.seg_start = (int *)(ws2 + o_seg);
        L.arr_of_pos = (int *)(ws2 + o_arr);
        L.seg_pos = (int *)(ws2 + o_pos);
        L.run_info = (int4 *)(ws2 + o_run);
        void *stage2 = ws2 + o_stage2;
        ANE_CUDA_TRY(cudaMemsetAsync(ws2, 0, o_zero_end, st));
        if (u16) eb_count_arrival_kernel<uint16_t><<<pb, 256, 0, st>>>(L, tokens, n, vocab, ctx().status);
        else eb_count_arrival_kernel<int32_t><<<pb, 256, 0, st>>>(L, tokens, n, vocab, ctx().status);
        eb_segments_kernel<<<(vocab + SEG_THREADS - 1) / SEG_THREADS, SEG_THREADS, 0, st>>>(L, vocab);
        const int TOKr = ER_WC * (esz == 2 ? 2 : 1);
        const int tps = (S + TOKr - 1) / TOKr;
        dim3 grid((unsigned)(B * tps), (unsigned)((D + ER_DC - 1) / ER_DC));
        const int rblocks = 8 * ctx().sm_count;
#define ANE_EB_SCATTER(Tv, ESZv, IDv)                                                                                                  \
        do {                                                                                                                          \
            eb_stage_rows_kernel<Tv, ESZv, IDv><<<grid, ER_THREADS, 0, st>>>(stage2, d_embed, dx, tokens, L.count, vocab, D, S, tps,  \
                                                                             L.seg_start, L.arr_of_pos, L.seg_pos);                   \
            eb_reduce_segments_kernel<Tv, ESZv, IDv><<<rblocks, RS_THREADS, 0, st>>>(d_embed, stage2, tokens, L, n, D);                \
        } while (0)
        if (dtype == ANE_F32) { if (u16) ANE_EB_SCATTER(float, 4, uint16_t); else ANE_EB_SCATTER(float, 4, int32_t); }
        else if (dtype == ANE_BF16) { if (u16) ANE_EB_SCATTER(__nv_bfloat16, 2, uint16_t); else ANE_EB_SCATTER(__nv_bfloat16, 2, int32_t); }
        else { if (u16) ANE_EB_SCATTER(__half, 2, uint16_t); else ANE_EB_SCATTER(__half, 2, int32_t); }
#undef ANE_EB_SCATTER
        ANE_LAUNCH_OK(4);
        return ANE_CUDA_OK;
    }

    size_t cub_bytes = 0;
    cub::DoubleBuffer<int> kb(nullptr, nullptr), vb(nullptr, nullptr);
    ANE_CUDA_TRY(cub::DeviceRadixSort::SortPairs(nullptr, cub_bytes, kb, vb, n, 0, sort_bits(vocab), st));
    const size_t off_k0 = 0, off_k1 = ints, off_v0 = 2 * ints, off_v1 = 3 * ints, off_aux = 4 * ints;   // aux: rank_of_pos or run_start
    const size_t off_cnt = 5 * ints;                                                                   // run_count, then count[vocab]
    const size_t off_cub = off_cnt + round_up(((size_t)vocab + 64) * sizeof(int), 256);
    const size_t off_stage = off_cub + round_up(cub_bytes, 256);
    const size_t total = off_stage + round_up((size_t)n * D * esz, 256);
    char *ws = static_cast<char *>(workspace(total));
    if (!ws) return fail(ANE_CUDA_ERR_NOMEM, "%s: no scratch (%zu bytes)", __func__, total);
    int *k0 = (int *)(ws + off_k0), *k1 = (int *)(ws + off_k1), *v0 = (int *)(ws + off_v0), *v1 = (int *)(ws + off_v1);
    int *aux = (int *)(ws + off_aux);
    void *stage = ws + off_stage;
    kb = cub::DoubleBuffer<int>(k0, k1);
    vb = cub::DoubleBuffer<int>(v0, v1);

    if (tiled) {
        EmbedSide *side = embed_side();
        if (!side) return fail(ANE_CUDA_ERR_CUDA, "%s: cannot create the side stream", __func__);
        int *run_count = (int *)(ws + off_cnt), *count = run_count + 64, *run_start = aux;
        ANE_CUDA_TRY(cudaMemsetAsync(run_count, 0, ((size_t)vocab + 64) * sizeof(int), st));
        // fork: keys -> sort -> run starts, beside the data movement
        ANE_CUDA_TRY(cudaEventRecord(side->fork, st));
        ANE_CUDA_TRY(cudaStreamWaitEvent(side->stream, side->fork, 0));
        if (u16) eb_keys_kernel<uint16_t><<<pb, 256, 0, side->stream>>>(k0, v0, tokens, n, vocab);
        else eb_keys_kernel<int32_t><<<pb, 256, 0, side->stream>>>(k0, v0, tokens, n, vocab);
        ANE_CUDA_TRY(cub::DeviceRadixSort::SortPairs(ws + off_cub, cub_bytes, kb, vb, n, 0, sort_bits(vocab), side->stream));
        eb_runs_kernel<<<pb, 256, 0, side->stream>>>(run_start, run_count, kb.Current(), n, vocab);
        ANE_CUDA_TRY(cudaEventRecord(side->join, side->stream));
        // main: occurrence counts, then every column to d_embed (single occurrence) or to its staging row
        if (u16) eb_count_kernel<uint16_t><<<pb, 256, 0, st>>>(count, tokens, n, vocab, ctx().status);
        else eb_count_kernel<int32_t><<<pb, 256, 0, st>>>(count, tokens, n, vocab, ctx().status);
        const int TOKr = ER_WC * (esz == 2 ? 2 : 1);
        const int tps = (S + TOKr - 1) / TOKr;
        dim3 grid((unsigned)(B * tps), (unsigned)((D + ER_DC - 1) / ER_DC));
        const int rblocks = ((n + 1) / 2 + RR_THREADS / 32 - 1) / (RR_THREADS / 32);   // a run has two positions or more
#define ANE_EB_ROWS(Tv, ESZv)                                                                                                         \
        do {                                                                                                                          \
            if (u16) eb_stage_rows_kernel<Tv, ESZv, uint16_t><<<grid, ER_THREADS, 0, st>>>(stage, d_embed, dx, tokens, count, vocab, D, S, tps, nullptr, nullptr, nullptr); \
            else eb_stage_rows_kernel<Tv, ESZv, int32_t><<<grid, ER_THREADS, 0, st>>>(stage, d_embed, dx, tokens, count, vocab, D, S, tps, nullptr, nullptr, nullptr);      \
            ANE_CUDA_TRY(cudaStreamWaitEvent(st, side->join, 0));                                                                     \
            eb_reduce_runs_kernel<Tv, ESZv><<<rblocks, RR_THREADS, 0, st>>>(d_embed, stage, kb.Current(), vb.Current(), run_start, run_count, n, D); \
        } while (0)
        if (dtype == ANE_F32) ANE_EB_ROWS(float, 4);
        else if (dtype == ANE_BF16) ANE_EB_ROWS(__nv_bfloat16, 2);
        else ANE_EB_ROWS(__half, 2);
#undef ANE_EB_ROWS
        ANE_LAUNCH_OK(5);
        return ANE_CUDA_OK;
    }

    // element-wise form for unaligned shapes
    if (u16) eb_prepare_kernel<uint16_t><<<pb, 256, 0, st>>>(k0, v0, tokens, n, vocab, ctx().status);
    else eb_prepare_kernel<int32_t><<<pb, 256, 0, st>>>(k0, v0, tokens, n, vocab, ctx().status);
    ANE_CUDA_TRY(cub::DeviceRadixSort::SortPairs(ws + off_cub, cub_bytes, kb, vb, n, 0, sort_bits(vocab), st));
    const int *keys = kb.Current();
    int *rank_of_pos = aux;
    eb_inverse_kernel<<<pb, 256, 0, st>>>(rank_of_pos, vb.Current(), n);
    if (dtype == ANE_F32) {
        constexpr int TT = 32, DC = 32;
        const int tps = (S + TT - 1) / TT;
        dim3 grid((unsigned)(B * tps), (unsigned)((D + DC - 1) / DC));
        eb_stage_kernel<uint32_t, TT, DC><<<grid, EMB_THREADS, 0, st>>>((uint32_t *)stage, (const uint32_t *)dx, rank_of_pos, D, S, tps);
        eb_reduce_kernel<float><<<n, 128, 0, st>>>(d_embed, (const float *)stage, keys, n, D, vocab);
    } else {
        constexpr int TT = 64, DC = 64;
        const int tps = (S + TT - 1) / TT;
        dim3 grid((unsigned)(B * tps), (unsigned)((D + DC - 1) / DC));
        eb_stage_kernel<uint16_t, TT, DC><<<grid, EMB_THREADS, 0, st>>>((uint16_t *)stage, (const uint16_t *)dx, rank_of_pos, D, S, tps);
        if (dtype == ANE_BF16) eb_reduce_kernel<__nv_bfloat16><<<n, 128, 0, st>>>(d_embed, (const __nv_bfloat16 *)stage, keys, n, D, vocab);
        else eb_reduce_kernel<__half><<<n, 128, 0, st>>>(d_embed, (const __half *)stage, keys, n, D, vocab);
    }
    ANE_LAUNCH_OK(4);
    return ANE_CUDA_OK;
}

}  // extern "C"
