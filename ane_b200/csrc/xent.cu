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

#include <math.h>

namespace ane {

constexpr int XE_THREADS = 256;
constexpr int XE_U = 4;

template <typename ID, int VEC, int LG>
__global__ void __launch_bounds__(XE_THREADS)
xent_kernel(float *dlogits, const float *logits, const void *__restrict__ targets, float *__restrict__ loss_tok,
            int V, int S, int tiles_per_seq, float grad_scale, ane_cuda_status *status) {
    constexpr int R = XE_THREADS / LG;
    constexpr int TW = LG * VEC;
    __shared__ float red_m[R][TW];
    __shared__ float red_s[R][TW];
    __shared__ float tot_m[TW];
    __shared__ float tot_is[TW];

    const int b = blockIdx.x / tiles_per_seq;
    const int lg = threadIdx.x % LG, rg = threadIdx.x / LG;
    const int t = (blockIdx.x % tiles_per_seq) * TW + lg * VEC;
    const bool active = t < S;
    const size_t base = (size_t)b * V * S + t;

    // sweep 1: online max / sum of exp
    float m[VEC], s[VEC];
#pragma unroll
    for (int j = 0; j < VEC; j++) { m[j] = -INFINITY; s[j] = 0.0f; }
    for (int vb = 0; vb < V; vb += R * XE_U) {
        Raw<float, VEC> r[XE_U];
        bool ok[XE_U];
#pragma unroll
        for (int u = 0; u < XE_U; u++) {
            const int v = vb + u * R + rg;
            ok[u] = active && v < V;
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
            if (gm[j] > m[j]) { s[j] = s[j] * expf(m[j] - gm[j]); m[j] = gm[j]; }   // exp(-inf) = 0 on the first group
        }
#pragma unroll
        for (int u = 0; u < XE_U; u++) {
            if (ok[u]) {
#pragma unroll
                for (int j = 0; j < VEC; j++) s[j] += expf(l[u][j] - m[j]);
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
        tot_m[threadIdx.x] = M;
        tot_is[threadIdx.x] = 1.0f / sum;                    // inv_sum, stories_cpu_ops.h:91-92
    }
    __syncthreads();

    float negM[VEC], inv[VEC];
    int tgt[VEC];
    const float invS = 1.0f / (float)S;
#pragma unroll
    for (int j = 0; j < VEC; j++) {
        negM[j] = -tot_m[lg * VEC + j];
        inv[j] = tot_is[lg * VEC + j];
        tgt[j] = -1;
        if (active) {
            const int id = (int)reinterpret_cast<const ID *>(targets)[(size_t)b * S + t + j];
            if (id >= 0 && id < V) tgt[j] = id;
            else if (rg == 0) {                                // one thread per token reports it
                atomicAdd(&status->oor_ids, 1);
                loss_tok[(size_t)b * S + t + j] = 0.0f;        // no loss term (stories_cpu_ops.h:98)
            }
        }
    }

    // sweep 2: p = exp(l - M) * inv_sum ; target row: loss and -1 ; then *1/S (and grad_scale)
    for (int vb = 0; vb < V; vb += R * XE_U) {
        Raw<float, VEC> r[XE_U];
        bool ok[XE_U];
#pragma unroll
        for (int u = 0; u < XE_U; u++) {
            const int v = vb + u * R + rg;
            ok[u] = active && v < V;
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
                    float p = expf(l[j] + negM[j]) * inv[j];
                    if (tgt[j] >= 0) {
                        if (v == tgt[j]) {
                            const float lt = -logf(p + 1e-10f);
                            loss_tok[(size_t)b * S + t + j] = lt;
                            if (!isfinite(lt)) atomicAdd(&status->nonfinite, 1);
                            p -= 1.0f;
                        }
                        p = p * invS;
                    }
                    if (grad_scale != 1.0f) p = p * grad_scale;
                    l[j] = p;
                }
                Raw<float, VEC> o;
                o.pack(l);
                o.store_stream(dlogits + base + (size_t)v * S);
            }
        }
    }
}

// ------------------------------------------------------------------ L2-resident wave kernel
// With V = 151936 one token's column is 608 KB: a token stripe does not fit on chip, and a block
// that sweeps its stripe twice reads it twice from HBM.  Here the WHOLE grid works on one "wave"
// of XW_W = 32 tokens (a 128-byte line per vocabulary row, 19 MB for V = 151936) at a time, each
// block owning a fixed slice of the vocabulary rows:
//   phase 1 (wave w)   stream the slice, online (max, sum) per token, block partial -> scratch;
//                      the last block to arrive merges all partials into (max, 1/sum) per token
//                      and raises flag[w];
//   phase 2 (wave w)   after flag[w]: stream the slice again -- still in L2, only about three
//                      waves (58 MB) are live at any time -- and write dlogits.
// Blocks run phase 1 of wave w+1 BEFORE phase 2 of wave w, so the merge of wave w is hidden
// behind real work and nobody idles at a grid-wide barrier.  The kernel is launched
// cooperatively (all blocks co-resident); the flag wait is bounded and reports a give-up in the
// status words instead of spinning forever.
constexpr int XW_THREADS = 256;
constexpr int XW_LG = 8;
constexpr int XW_VEC = 4;
constexpr int XW_W = XW_LG * XW_VEC;      // 32 tokens per wave
constexpr int XW_R = XW_THREADS / XW_LG;  // 32 vocabulary rows per sweep step
constexpr int XW_U = 4;
constexpr int XW_BUFS = 3;

struct XentWaveScratch {
    float2 *partial;     // [XW_BUFS][grid][XW_W]  (max, sum) per block and token
    float2 *final_ms;    // [XW_BUFS][XW_W]        (max, 1/sum) per token
    unsigned *counter;   // [nwaves] blocks arrived
    unsigned *flag;      // [nwaves] merged
};

template <typename ID>
__global__ void __launch_bounds__(XW_THREADS)
xent_wave_kernel(float *dlogits, const float *logits, const void *__restrict__ targets, float *__restrict__ loss_tok,
                 int V, int S, int waves_per_seq, int nwaves, float grad_scale, XentWaveScratch sc, ane_cuda_status *status) {
    __shared__ __align__(16) float red_m[XW_R][XW_W];
    __shared__ __align__(16) float red_s[XW_R][XW_W];
    __shared__ float mrg_m[XW_THREADS / 32][XW_W];
    __shared__ float mrg_s[XW_THREADS / 32][XW_W];
    __shared__ int is_last, give_up;

    const int G = gridDim.x;
    const int lg = threadIdx.x % XW_LG, rg = threadIdx.x / XW_LG;
    const int rows_per = (V + G - 1) / G;
    const int v0 = blockIdx.x * rows_per;
    const int v1 = v0 + rows_per < V ? v0 + rows_per : V;
    const float invS = 1.0f / (float)S;
    if (threadIdx.x == 0) give_up = 0;
    __syncthreads();

    for (int w = 0; w <= nwaves; w++) {
        // ---------------- phase 1 of wave w
        if (w < nwaves) {
            const int b = w / waves_per_seq;
            const int t = (w % waves_per_seq) * XW_W + lg * XW_VEC;
            const bool active = t < S;
            const size_t base = (size_t)b * V * S + t;
            float m[XW_VEC], s[XW_VEC];
#pragma unroll
            for (int j = 0; j < XW_VEC; j++) { m[j] = -INFINITY; s[j] = 0.0f; }
            for (int vb = v0; vb < v1; vb += XW_R * XW_U) {
                float4 r[XW_U];
                bool ok[XW_U];
#pragma unroll
                for (int u = 0; u < XW_U; u++) {
                    const int v = vb + u * XW_R + rg;
                    ok[u] = active && v < v1;
                    if (ok[u]) r[u] = *reinterpret_cast<const float4 *>(logits + base + (size_t)v * S);   // stays in L2 for phase 2
                }
                float gm[XW_VEC];
#pragma unroll
                for (int j = 0; j < XW_VEC; j++) gm[j] = m[j];
#pragma unroll
                for (int u = 0; u < XW_U; u++)
                    if (ok[u]) {
                        gm[0] = fmaxf(gm[0], r[u].x); gm[1] = fmaxf(gm[1], r[u].y);
                        gm[2] = fmaxf(gm[2], r[u].z); gm[3] = fmaxf(gm[3], r[u].w);
                    }
#pragma unroll
                for (int j = 0; j < XW_VEC; j++)
                    if (gm[j] > m[j]) { s[j] = s[j] * expf(m[j] - gm[j]); m[j] = gm[j]; }
#pragma unroll
                for (int u = 0; u < XW_U; u++)
                    if (ok[u]) {
                        s[0] += expf(r[u].x - m[0]); s[1] += expf(r[u].y - m[1]);
                        s[2] += expf(r[u].z - m[2]); s[3] += expf(r[u].w - m[3]);
                    }
            }
            *reinterpret_cast<float4 *>(&red_m[rg][lg * XW_VEC]) = make_float4(m[0], m[1], m[2], m[3]);
            *reinterpret_cast<float4 *>(&red_s[rg][lg * XW_VEC]) = make_float4(s[0], s[1], s[2], s[3]);
            __syncthreads();
            if (threadIdx.x < XW_W) {
                float M = -INFINITY;
                for (int q = 0; q < XW_R; q++) M = fmaxf(M, red_m[q][threadIdx.x]);
                float sum = 0.0f;
                for (int q = 0; q < XW_R; q++) {
                    const float mq = red_m[q][threadIdx.x];
                    if (mq > -INFINITY) sum += red_s[q][threadIdx.x] * expf(mq - M);
                }
                sc.partial[((size_t)(w % XW_BUFS) * G + blockIdx.x) * XW_W + threadIdx.x] = make_float2(M, sum);
                __threadfence();
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                const unsigned ticket = atomicAdd(&sc.counter[w], 1u);
                is_last = ticket == (unsigned)(G - 1);
                if (is_last) __threadfence();
            }
            __syncthreads();
            if (is_last) {      // merge the G partials of every token: warp `part` takes blocks part, part+8, ...
                const int tok = threadIdx.x % XW_W, part = threadIdx.x / XW_W;
                constexpr int PARTS = XW_THREADS / XW_W;
                const float2 *pp = sc.partial + (size_t)(w % XW_BUFS) * G * XW_W;
                float M = -INFINITY;
                for (int i = part; i < G; i += PARTS) M = fmaxf(M, __ldcg(&pp[(size_t)i * XW_W + tok]).x);
                mrg_m[part][tok] = M;
                __syncthreads();
                M = -INFINITY;
#pragma unroll
                for (int q = 0; q < PARTS; q++) M = fmaxf(M, mrg_m[q][tok]);
                float sum = 0.0f;
                for (int i = part; i < G; i += PARTS) {
                    const float2 ms = __ldcg(&pp[(size_t)i * XW_W + tok]);
                    if (ms.x > -INFINITY) sum += ms.y * expf(ms.x - M);
                }
                mrg_s[part][tok] = sum;
                __syncthreads();
                if (part == 0) {
                    sum = 0.0f;
#pragma unroll
                    for (int q = 0; q < PARTS; q++) sum += mrg_s[q][tok];
                    sc.final_ms[(w % XW_BUFS) * XW_W + tok] = make_float2(M, 1.0f / sum);     // inv_sum, stories_cpu_ops.h:91-92
                    __threadfence();
                }
                __syncthreads();
                if (threadIdx.x == 0) atomicExch(&sc.flag[w], 1u);
            }
        }
        // ---------------- phase 2 of wave w-1
        if (w >= 1) {
            const int pw = w - 1;
            if (threadIdx.x == 0) {
                unsigned spins = 0;
                while (atomicAdd(&sc.flag[pw], 0u) == 0u) {
                    __nanosleep(64);
                    if (++spins > (1u << 22)) { give_up = 1; break; }
                }
                __threadfence();
            }
            __syncthreads();
            if (give_up) {
                if (threadIdx.x == 0) atomicAdd(&status->wait_giveups, 1);
                return;
            }
            const int b = pw / waves_per_seq;
            const int t = (pw % waves_per_seq) * XW_W + lg * XW_VEC;
            const bool active = t < S;
            const size_t base = (size_t)b * V * S + t;
            float negM[XW_VEC], inv[XW_VEC];
            int tgt[XW_VEC];
#pragma unroll
            for (int j = 0; j < XW_VEC; j++) {
                const float2 ms = __ldcg(&sc.final_ms[(pw % XW_BUFS) * XW_W + lg * XW_VEC + j]);
                negM[j] = -ms.x;
                inv[j] = ms.y;
                tgt[j] = -1;
                if (active) {
                    const int id = (int)reinterpret_cast<const ID *>(targets)[(size_t)b * S + t + j];
                    if (id >= 0 && id < V) tgt[j] = id;
                    else if (rg == 0 && blockIdx.x == 0) {        // one thread per token reports it
                        atomicAdd(&status->oor_ids, 1);
                        loss_tok[(size_t)b * S + t + j] = 0.0f;   // no loss term (stories_cpu_ops.h:98)
                    }
                }
            }
            for (int vb = v0; vb < v1; vb += XW_R * XW_U) {
                float4 r[XW_U];
                bool ok[XW_U];
#pragma unroll
                for (int u = 0; u < XW_U; u++) {
                    const int v = vb + u * XW_R + rg;
                    ok[u] = active && v < v1;
                    if (ok[u]) r[u] = __ldcs(reinterpret_cast<const float4 *>(logits + base + (size_t)v * S));
                }
#pragma unroll
                for (int u = 0; u < XW_U; u++) {
                    const int v = vb + u * XW_R + rg;
                    if (ok[u]) {
                        float l[XW_VEC] = {r[u].x, r[u].y, r[u].z, r[u].w};
#pragma unroll
                        for (int j = 0; j < XW_VEC; j++) {
                            float p = expf(l[j] + negM[j]) * inv[j];
                            if (tgt[j] >= 0) {
                                if (v == tgt[j]) {
                                    const float lt = -logf(p + 1e-10f);
                                    loss_tok[(size_t)b * S + t + j] = lt;
                                    if (!isfinite(lt)) atomicAdd(&status->nonfinite, 1);
                                    p -= 1.0f;
                                }
                                p = p * invS;
                            }
                            if (grad_scale != 1.0f) p = p * grad_scale;
                            l[j] = p;
                        }
                        __stcs(reinterpret_cast<float4 *>(dlogits + base + (size_t)v * S), make_float4(l[0], l[1], l[2], l[3]));
                    }
                }
            }
        }
    }
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

extern "C" {

int ane_cuda_cross_entropy_dev(void *stream, ane_idtype idtype, int B, int V, int S, float *dlogits, const float *logits,
                               const void *targets, float *loss_seq, float grad_scale) {
    ANE_REQUIRE_INIT();
    ANE_REQUIRE(dlogits && logits && targets && loss_seq, "%s: null pointer", __func__);
    ANE_REQUIRE(idtype == ANE_ID_U16 || idtype == ANE_ID_I32, "%s: bad id type", __func__);
    ANE_REQUIRE(B >= 1 && V >= 1 && S >= 1, "%s: bad shape B=%d V=%d S=%d", __func__, B, V, S);
    ANE_REQUIRE((long long)B * S < 0x7fffffffLL, "%s: too many tokens", __func__);
    cudaStream_t st = (cudaStream_t)stream;
    float *loss_tok = static_cast<float *>(workspace((size_t)B * S * sizeof(float)));
    if (!loss_tok) return fail(ANE_CUDA_ERR_NOMEM, "%s: no scratch", __func__);
    ane_cuda_status *status = ctx().status;
    const bool vec = (S % 4 == 0) && aligned16(dlogits) && aligned16(logits);
    if (vec && tuning("xent_wave", 1) && V >= 8192 && (long long)B * S >= 1024) {
        // whole-grid waves of 32 tokens kept in L2 between the two sweeps (cooperative launch)
        int per_sm = 0;
        auto kern = idtype == ANE_ID_U16 ? xent_wave_kernel<uint16_t> : xent_wave_kernel<int32_t>;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, XW_THREADS, 0) == cudaSuccess && per_sm >= 1) {
            if (per_sm > 2) per_sm = 2;
            int G = per_sm * ctx().sm_count;
            const int wps = (S + XW_W - 1) / XW_W;
            int nwaves = B * wps;
            const size_t off_part = round_up((size_t)B * S * sizeof(float), 256);
            const size_t off_final = off_part + round_up((size_t)XW_BUFS * G * XW_W * sizeof(float2), 256);
            const size_t off_cnt = off_final + round_up((size_t)XW_BUFS * XW_W * sizeof(float2), 256);
            const size_t off_flag = off_cnt + round_up((size_t)nwaves * sizeof(unsigned), 256);
            const size_t total = off_flag + round_up((size_t)nwaves * sizeof(unsigned), 256);
            char *ws = static_cast<char *>(workspace(total));
            if (!ws) return fail(ANE_CUDA_ERR_NOMEM, "%s: no scratch", __func__);
            loss_tok = reinterpret_cast<float *>(ws);
            XentWaveScratch sc;
            sc.partial = reinterpret_cast<float2 *>(ws + off_part);
            sc.final_ms = reinterpret_cast<float2 *>(ws + off_final);
            sc.counter = reinterpret_cast<unsigned *>(ws + off_cnt);
            sc.flag = reinterpret_cast<unsigned *>(ws + off_flag);
            ANE_CUDA_TRY(cudaMemsetAsync(ws + off_cnt, 0, total - off_cnt, st));
            void *args[] = {&dlogits, &logits, &targets, &loss_tok, &V, &S, (void *)&wps, &nwaves, &grad_scale, &sc, &status};
            ANE_CUDA_TRY(cudaLaunchCooperativeKernel((const void *)kern, dim3(G), dim3(XW_THREADS), args, 0, st));
            xent_loss_kernel<<<B, 256, 0, st>>>(loss_seq, loss_tok, S);
            ANE_LAUNCH_OK(2);
            return ANE_CUDA_OK;
        }
    }
    if (vec) {
        constexpr int LG = 8, VEC = 4;
        const int tps = (S + LG * VEC - 1) / (LG * VEC);
        const unsigned grid = (unsigned)(B * tps);
        if (idtype == ANE_ID_U16) xent_kernel<uint16_t, VEC, LG><<<grid, XE_THREADS, 0, st>>>(dlogits, logits, targets, loss_tok, V, S, tps, grad_scale, status);
        else xent_kernel<int32_t, VEC, LG><<<grid, XE_THREADS, 0, st>>>(dlogits, logits, targets, loss_tok, V, S, tps, grad_scale, status);
    } else {
        constexpr int LG = 32, VEC = 1;
        const int tps = (S + LG - 1) / LG;
        const unsigned grid = (unsigned)(B * tps);
        if (idtype == ANE_ID_U16) xent_kernel<uint16_t, VEC, LG><<<grid, XE_THREADS, 0, st>>>(dlogits, logits, targets, loss_tok, V, S, tps, grad_scale, status);
        else xent_kernel<int32_t, VEC, LG><<<grid, XE_THREADS, 0, st>>>(dlogits, logits, targets, loss_tok, V, S, tps, grad_scale, status);
    }
    xent_loss_kernel<<<B, 256, 0, st>>>(loss_seq, loss_tok, S);
    ANE_LAUNCH_OK(2);
    return ANE_CUDA_OK;
}

}  // extern "C"
