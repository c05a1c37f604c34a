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
    cudaStream_t st = (cudaStream_t)stream;
    const bool zero = flags == ANE_OOR_ZERO;
    ane_cuda_status *status = ctx().status;
    if (dtype == ANE_F32) {
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
    cudaStream_t st = (cudaStream_t)stream;
    const int n = B * S;
    const size_t esz = dtype_size(dtype);

    size_t cub_bytes = 0;
    cub::DoubleBuffer<int> kb(nullptr, nullptr), vb(nullptr, nullptr);
    ANE_CUDA_TRY(cub::DeviceRadixSort::SortPairs(nullptr, cub_bytes, kb, vb, n, 0, sort_bits(vocab), st));
    const size_t ints = round_up((size_t)n * sizeof(int), 256);
    const size_t off_k0 = 0, off_k1 = ints, off_v0 = 2 * ints, off_v1 = 3 * ints, off_rank = 4 * ints;
    const size_t off_cub = 5 * ints;
    const size_t off_stage = off_cub + round_up(cub_bytes, 256);
    const size_t total = off_stage + round_up((size_t)n * D * esz, 256);
    char *ws = static_cast<char *>(workspace(total));
    if (!ws) return fail(ANE_CUDA_ERR_NOMEM, "%s: no scratch (%zu bytes)", __func__, total);
    int *k0 = (int *)(ws + off_k0), *k1 = (int *)(ws + off_k1), *v0 = (int *)(ws + off_v0), *v1 = (int *)(ws + off_v1);
    int *rank_of_pos = (int *)(ws + off_rank);

    const int pb = (n + 255) / 256;
    if (idtype == ANE_ID_U16) eb_prepare_kernel<uint16_t><<<pb, 256, 0, st>>>(k0, v0, tokens, n, vocab, ctx().status);
    else eb_prepare_kernel<int32_t><<<pb, 256, 0, st>>>(k0, v0, tokens, n, vocab, ctx().status);
    kb = cub::DoubleBuffer<int>(k0, k1);
    vb = cub::DoubleBuffer<int>(v0, v1);
    ANE_CUDA_TRY(cub::DeviceRadixSort::SortPairs(ws + off_cub, cub_bytes, kb, vb, n, 0, sort_bits(vocab), st));
    const int *keys = kb.Current();
    const int *sorted_pos = vb.Current();
    eb_inverse_kernel<<<pb, 256, 0, st>>>(rank_of_pos, sorted_pos, n);
    if (dtype == ANE_F32) {
        constexpr int TT = 32, DC = 32;
        const int tps = (S + TT - 1) / TT;
        dim3 grid((unsigned)(B * tps), (unsigned)((D + DC - 1) / DC));
        eb_stage_kernel<uint32_t, TT, DC><<<grid, EMB_THREADS, 0, st>>>((uint32_t *)(ws + off_stage), (const uint32_t *)dx, rank_of_pos, D, S, tps);
        eb_reduce_kernel<float><<<n, 128, 0, st>>>(d_embed, (const float *)(ws + off_stage), keys, n, D, vocab);
    } else {
        constexpr int TT = 64, DC = 64;
        const int tps = (S + TT - 1) / TT;
        dim3 grid((unsigned)(B * tps), (unsigned)((D + DC - 1) / DC));
        eb_stage_kernel<uint16_t, TT, DC><<<grid, EMB_THREADS, 0, st>>>((uint16_t *)(ws + off_stage), (const uint16_t *)dx, rank_of_pos, D, S, tps);
        if (dtype == ANE_BF16)
            eb_reduce_kernel<__nv_bfloat16><<<n, 128, 0, st>>>(d_embed, (const __nv_bfloat16 *)(ws + off_stage), keys, n, D, vocab);
        else
            eb_reduce_kernel<__half><<<n, 128, 0, st>>>(d_embed, (const __half *)(ws + off_stage), keys, n, D, vocab);
    }
    ANE_LAUNCH_OK(4);
    return ANE_CUDA_OK;
}

}  // extern "C"
