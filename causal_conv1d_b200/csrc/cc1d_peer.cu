// One-shot all-reduce of the packed fp32 weight-gradient buffer over peer memory (sm_100a, NVLink).
//
// The batch-sharded backward ends with a sum over ranks of at most a few hundred KB (dim * (width
// + 1) floats).  At that size a ring or tree is all latency; here every rank stores its partial
// straight into a slot of every peer's exchange buffer (plain peer stores), raises a flag next to
// it, waits for the flags of all peers in its own buffer and adds the world's slots in rank
// order — one kernel, one NVLink crossing, and the same bits on every rank because the order of
// the additions is fixed.  No multicast, no loads from peer memory: peers only ever WRITE into
// each other's buffers, every read is local.
//
// Exchange buffer of a rank (same layout on all ranks, allocated by the caller as peer-mapped
// memory and zero-filled once):
//   [0, kPeerFlagBytes)   uint32 flags[2][kMaxPeers][kPeerCtas]   flag = epoch of the data beside it
//   then                  float  slots[2][world][count]
// Two parities alternate with the epoch, so a rank that is one call ahead never overwrites data a
// slower rank is still adding up (it cannot get two ahead: its next call needs this rank's flags).
// The vector is cut into kPeerCtas slices; CTA c moves, flags, awaits and adds slice c only, so
// CTAs never wait for each other.  Every wait is bounded: when it runs out the CTA sets *status
// and leaves dst untouched.
#include "cc1d_common.cuh"
#include "cc1d_kernels.h"

namespace cc1d {

constexpr int kMaxPeers = CC1D_MAX_PEERS;
constexpr int kPeerCtas = 8;
constexpr int kPeerThreads = 256;
constexpr size_t kPeerFlagBytes = 4096;
static_assert(2 * kMaxPeers * kPeerCtas * sizeof(uint32_t) <= kPeerFlagBytes, "flag area too small");
constexpr uint32_t kPeerSpinLimit = 1u << 21;   // x ~0.25 us of sleep: about half a second

struct PeerArgs {
    const float *src;
    float *dst;
    char *base[kMaxPeers];    // base[r]: rank r's exchange buffer as seen from this device
    int *status;
    int64_t count;            // floats, a multiple of 4
    int world, rank;
    uint32_t epoch;
};

__device__ __forceinline__ uint32_t *peer_flag(char *base, uint32_t parity, int from_rank, int cta) {
    return reinterpret_cast<uint32_t *>(base) + (parity * kMaxPeers + from_rank) * kPeerCtas + cta;
}
__device__ __forceinline__ float4 *peer_slot(char *base, uint32_t parity, int from_rank, int world, int64_t count) {
    return reinterpret_cast<float4 *>(base + kPeerFlagBytes) + ((int64_t)parity * world + from_rank) * (count / 4);
}

__global__ void __launch_bounds__(kPeerThreads) peer_allreduce_kernel(const PeerArgs a) {
    pdl_wait();
    __shared__ int s_expired;
    const uint32_t parity = a.epoch & 1u;
    const int64_t nvec = a.count / 4;
    const int64_t per = (nvec + kPeerCtas - 1) / kPeerCtas;
    const int64_t v0 = (int64_t)blockIdx.x * per, v1 = v0 + per < nvec ? v0 + per : nvec;
    if (threadIdx.x == 0) s_expired = 0;

    // 1. this rank's slice into every rank's slot (own slot included), then the flags
    const float4 *src = reinterpret_cast<const float4 *>(a.src);
    for (int64_t v = v0 + threadIdx.x; v < v1; v += kPeerThreads) {
        const float4 val = src[v];
        for (int r = 0; r < a.world; ++r) peer_slot(a.base[r], parity, a.rank, a.world, a.count)[v] = val;
    }
    __threadfence_system();       // this thread's peer stores are visible system-wide ...
    __syncthreads();              // ... for every thread of the CTA, before the flags go out
    if ((int)threadIdx.x < a.world) {
        uint32_t *f = peer_flag(a.base[threadIdx.x], parity, a.rank, blockIdx.x);
        asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(f), "r"(a.epoch) : "memory");
    }

    // 2. wait (bounded) until every rank's slice c has landed in this rank's buffer
    if ((int)threadIdx.x < a.world) {
        const uint32_t *f = peer_flag(a.base[a.rank], parity, threadIdx.x, blockIdx.x);
        uint32_t seen = 0, it = 0;
        for (; it < kPeerSpinLimit; ++it) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(f) : "memory");
            if (seen == a.epoch) break;
            __nanosleep(it < 64 ? 20 : 250);
        }
        if (seen != a.epoch) s_expired = 1;
    }
    __syncthreads();
    if (s_expired) {              // give up: report, leave dst as it is
        if (threadIdx.x == 0) *a.status = 1;
        return;
    }
    __threadfence_system();

    // 3. add the world's slots in rank order (local reads only)
    float4 *dst = reinterpret_cast<float4 *>(a.dst);
    for (int64_t v = v0 + threadIdx.x; v < v1; v += kPeerThreads) {
        float4 acc = __ldcv(peer_slot(a.base[a.rank], parity, 0, a.world, a.count) + v);
        for (int r = 1; r < a.world; ++r) {
            const float4 t = __ldcv(peer_slot(a.base[a.rank], parity, r, a.world, a.count) + v);
            acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
        }
        dst[v] = acc;
    }
}

size_t peer_allreduce_buffer_bytes(int world, int64_t count) {
    if (world < 1 || world > kMaxPeers || count < 0) return 0;
    const int64_t padded = (count + 3) / 4 * 4;
    return kPeerFlagBytes + (size_t)2 * (size_t)world * (size_t)padded * sizeof(float);
}

int launch_peer_allreduce(const cc1d_peer_allreduce_params &p, cudaStream_t stream) {
    PeerArgs a;
    a.src = p.src; a.dst = p.dst; a.status = p.status;
    a.count = p.count; a.world = p.world; a.rank = p.rank; a.epoch = p.epoch;
    for (int r = 0; r < kMaxPeers; ++r) a.base[r] = r < p.world ? reinterpret_cast<char *>(p.peer_base[r]) : nullptr;
    launch_k(peer_allreduce_kernel, dim3(kPeerCtas), dim3(kPeerThreads), 0, stream, a);
    return check_launch();
}

}  // namespace cc1d
