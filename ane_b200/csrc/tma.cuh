// tma.cuh -- thin wrappers around the Blackwell/Hopper bulk tensor copy engine (TMA) and the
// shared-memory transaction barriers (mbarrier) it signals.  Only what the kernels here need:
// 3-D tiled loads global -> shared memory of the issuing CTA, barrier init / expect-tx /
// bounded parity wait.
#pragma once

#include <cuda.h>          // CUtensorMap and its enums (types only: the encoder is resolved at run time)
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace ane {

// ------------------------------------------------------------------ host: tensor-map encoding
// [B][C][S] tensor of `dtype` elements seen as a 3-D map (S innermost); the box is
// box_s tokens x box_c channels x 1 sequence.  Requirements checked here: 16-byte aligned base,
// S*elt a multiple of 16 bytes, box_s*elt a multiple of 16 bytes, box dims <= 256.
// l2_promotion_bytes (0, 64, 128, 256): granularity the copy engine may widen L2 fills to; keep it no
// wider than a box row, or every row costs a wider DRAM fetch than it uses.
int make_bcs_tensor_map(CUtensorMap *map, ane_dtype dtype, const void *base, int B, int C, int S, int box_s, int box_c,
                        int l2_promotion_bytes = 128);

#ifdef __CUDACC__
// ------------------------------------------------------------------ device primitives
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// Make barrier initialisation visible to the async proxy before the first TMA uses it.
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// Order this thread's earlier generic-proxy accesses to shared memory before later async-proxy ones.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: every try_wait suspends the thread for a hardware-defined time slice, so the
// limit below is far beyond any legitimate copy latency (several milliseconds at least) and still
// finite.  Returns false when it gave up.
constexpr uint32_t MBAR_WAIT_LIMIT = 1u << 20;
// Test hook of the ring kernels (tuning knobs "qk_test_skip_item", "qk_wait_limit"): the producer arms the barrier of
// one work item but issues no copy for it, so that the consumer's bounded wait runs out -- the give-up path can be
// exercised without any fault.  skip_item < 0: off.
struct RingTest { int skip_item; uint32_t wait_limit; };
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint32_t limit = MBAR_WAIT_LIMIT) {
    for (uint32_t i = 0; i < limit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// Tiled 3-D load: box at coordinates (x = token, y = channel, z = sequence) -> dst (shared,
// 128-byte aligned); completion is signalled on `bar` as transferred bytes.  x * element size
// must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, int x, int y, int z, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}
#endif  // __CUDACC__

}  // namespace ane
