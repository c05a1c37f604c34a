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
