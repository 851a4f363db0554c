// TMA (cp.async.bulk.tensor) + mbarrier helpers for the channel-last kernels (sm_100a).
//
// The channel-last tensors are walked token by token; a warp owns a strip of 128 channels (256
// or 512 bytes wide).  Instead of holding the in-flight loads in registers, one lane of the warp
// asks the TMA unit for a box of [kTmaRows tokens x strip] into shared memory and every lane then
// reads its 8 or 16 bytes per token with ld.shared.  Bytes in flight are bounded by shared memory,
// not by registers or occupancy.  No multicast, no cluster: every box is this GPU's own memory
// going to this CTA's own shared memory.
#pragma once

#include <cuda.h>   // CUtensorMap and the cuTensorMapEncodeTiled prototype (resolved at run time)
#include <cuda_runtime.h>
#include <stdint.h>

namespace cc1d {

constexpr int kTmaRows = 8;          // tokens per box
constexpr int kTmaRowBytes = 512;    // default strip width: 32 lanes x 16 bytes
constexpr int kTmaStageBytes = kTmaRows * kTmaRowBytes;
constexpr uint32_t kTmaSpinLimit = 1u << 22;   // bounded wait: try_wait attempts before giving up

// Set by a kernel of this translation unit whose bounded mbarrier wait ran out (never expected).
// One copy per translation unit; read_and_clear_wait_expired() (below) is how the host sees it.
static __device__ int g_tma_wait_expired;

// Host: value of this translation unit's flag on the current device, reset to 0.  Synchronises.
static inline int read_and_clear_wait_expired() {
    int v = 0;
    const int zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_tma_wait_expired, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) (void)cudaMemcpyToSymbol(g_tma_wait_expired, &zero, sizeof(int));
    return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
// make mbarrier initialisation visible to the async (TMA) proxy
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// order this thread's earlier generic-proxy accesses to shared memory before later async-proxy ones
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
// Bounded wait on a phase parity.  Returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kTmaSpinLimit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// 3-D tiled load: box at (c0, c1, c2) of the tensor map -> shared memory, completion on `bar`.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        :: "r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" :: "l"(map) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// Host: tensor map over a channel-last tensor (dim, seqlen, batch) with element strides
// (1, l_stride, batch_stride) and a box of [row_bytes of channels, kTmaRows tokens, 1].
// Returns false when the driver entry point is missing or the encode is rejected (the
// caller then uses the non-TMA kernel).
bool make_channel_last_tensor_map(CUtensorMap *map, int dtype, const void *base, int64_t dim, int64_t seqlen,
                                  int64_t batch, int64_t l_stride, int64_t batch_stride, int row_bytes = kTmaRowBytes);

// Host: tensor map over a channel-first tensor (seqlen, dim, batch) with element strides
// (1, c_stride, batch_stride) and a box of [box_tokens tokens, box_channels channels, 1]: the box
// lands in shared memory channel by channel, box_tokens elements each.
bool make_channel_first_tensor_map(CUtensorMap *map, int dtype, const void *base, int64_t seqlen, int64_t dim,
                                   int64_t batch, int64_t c_stride, int64_t batch_stride, int box_tokens, int box_channels);

}  // namespace cc1d
