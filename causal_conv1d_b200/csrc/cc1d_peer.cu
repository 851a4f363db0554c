// One-shot all-reduce of the packed fp32 weight-gradient buffer over peer memory (sm_100a, NVLink).
//
// The batch-sharded backward ends with a sum over ranks of at most a few hundred KB (dim * (width
// + 1) floats).  At that size a ring or tree is all latency; here every rank stores its partial
// straight into a slot of every peer's exchange buffer (plain peer stores), every rank then reads
// the world's slots out of its OWN buffer and adds them in rank order — one kernel, one NVLink
// crossing, and the same bits on every rank because the order of the additions is fixed.  No
// multicast, no loads from peer memory: peers only ever WRITE into each other's buffers.
//
// There is no separate flag and no memory fence: data travels in 16-byte lines
//     { value[2i], epoch, value[2i+1], epoch }
// written with one 16-byte store; each 8-byte half carries its own epoch stamp, so a reader that
// polls a line until both stamps equal the current epoch has the data, whatever order the lines
// arrive in (the scheme NCCL calls LL).  Twice the bytes, none of the fence latency.
//
// Exchange buffer of a rank (same layout on all ranks, allocated by the caller as peer-mapped
// memory and zero-filled once):
//   [0, kPeerHeaderBytes)  uint32 calls[kPeerCtas]                collectives done so far (see below)
//   then                   uint4  lines[2][world][count / 2]
// Two parities alternate with the epoch, so a rank that is one call ahead never overwrites lines a
// slower rank has yet to read (it cannot get two ahead: its next call needs this rank's lines).
// The epoch of a collective is either given by the caller or (epoch == 0) taken from the rank's
// own `calls` words, which the kernel advances itself — a captured CUDA graph can then be replayed
// any number of times and every replay is a new collective.
// Every poll is bounded (spin_limit polls): when it runs out the thread sets *status, writes NaN to
// the elements it could not complete and stops.
#include "cc1d_common.cuh"
#include "cc1d_kernels.h"

namespace cc1d {

constexpr int kMaxPeers = CC1D_MAX_PEERS;
constexpr int kPeerCtas = 8;
constexpr int kPeerThreads = 256;
constexpr size_t kPeerHeaderBytes = 4096;
constexpr uint32_t kPeerSpinLimit = 1u << 21;   // x ~0.25 us of sleep: about half a second

struct PeerArgs {
    const float *src;
    float *dst;
    char *base[kMaxPeers];    // base[r]: rank r's exchange buffer as seen from this device
    int *status;
    int64_t count;            // floats, a multiple of 4
    int world, rank;
    uint32_t epoch;           // 0: numbered by the kernel
    uint32_t spin_limit;
};

__device__ __forceinline__ uint4 *peer_lines(char *base, uint32_t parity, int from_rank, int world, int64_t count) {
    return reinterpret_cast<uint4 *>(base + kPeerHeaderBytes) + ((int64_t)parity * world + from_rank) * (count / 2);
}
__device__ __forceinline__ void st_line(uint4 *p, const uint4 &v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_line(const uint4 *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kPeerThreads) peer_allreduce_kernel(const PeerArgs a) {
    pdl_wait();
    __shared__ uint32_t s_epoch;
    uint32_t *calls = reinterpret_cast<uint32_t *>(a.base[a.rank]) + blockIdx.x;   // the CTA's own word
    if (threadIdx.x == 0) {
        s_epoch = a.epoch != 0 ? a.epoch : *calls + 1;
        if (a.epoch == 0) *calls = s_epoch;
    }
    __syncthreads();
    const uint32_t epoch = s_epoch;
    const uint32_t parity = epoch & 1u;
    const int64_t nline = a.count / 2;
    const int64_t i0 = (int64_t)blockIdx.x * kPeerThreads + threadIdx.x, step = (int64_t)kPeerCtas * kPeerThreads;

    // 1. this rank's values, stamped, into every rank's buffer (own buffer included)
    const float2 *src = reinterpret_cast<const float2 *>(a.src);
    for (int64_t i = i0; i < nline; i += step) {
        const float2 v = src[i];
        const uint4 line = make_uint4(__float_as_uint(v.x), epoch, __float_as_uint(v.y), epoch);
        for (int r = 0; r < a.world; ++r) st_line(peer_lines(a.base[r], parity, a.rank, a.world, a.count) + i, line);
    }
    // 2. the world's lines out of this rank's buffer, added in rank order
    float2 *dst = reinterpret_cast<float2 *>(a.dst);
    for (int64_t i = i0; i < nline; i += step) {
        float2 acc = make_float2(0.f, 0.f);
        for (int r = 0; r < a.world; ++r) {
            const uint4 *p = peer_lines(a.base[a.rank], parity, r, a.world, a.count) + i;
            uint4 line = ld_line(p);
            for (uint32_t it = 0; (line.y != epoch || line.w != epoch) && it < a.spin_limit; ++it) {
                __nanosleep(it < 64 ? 20 : 250);
                line = ld_line(p);
            }
            if (line.y != epoch || line.w != epoch) {
                // the peer never delivered: report, and poison this and every remaining element of
                // this thread so that a caller who never reads the status cannot use the sums
                *a.status = 1;
                const float nan = __uint_as_float(0x7fc00000u);
                for (int64_t k = i; k < nline; k += step) dst[k] = make_float2(nan, nan);
                return;
            }
            if (r == 0) acc = make_float2(__uint_as_float(line.x), __uint_as_float(line.z));
            else { acc.x += __uint_as_float(line.x); acc.y += __uint_as_float(line.z); }
        }
        dst[i] = acc;
    }
}

size_t peer_allreduce_buffer_bytes(int world, int64_t count) {
    if (world < 1 || world > kMaxPeers || count < 0) return 0;
    const int64_t padded = (count + 3) / 4 * 4;
    return kPeerHeaderBytes + (size_t)2 * (size_t)world * (size_t)(padded / 2) * sizeof(uint4);
}

int launch_peer_allreduce(const cc1d_peer_allreduce_params &p, cudaStream_t stream) {
    PeerArgs a;
    a.src = p.src; a.dst = p.dst; a.status = p.status;
    a.count = p.count; a.world = p.world; a.rank = p.rank; a.epoch = p.epoch;
    a.spin_limit = p.spin_limit != 0 ? p.spin_limit : kPeerSpinLimit;
    for (int r = 0; r < kMaxPeers; ++r) a.base[r] = r < p.world ? reinterpret_cast<char *>(p.peer_base[r]) : nullptr;
    launch_k(peer_allreduce_kernel, dim3(kPeerCtas), dim3(kPeerThreads), 0, stream, a);
    return check_launch();
}

}  // namespace cc1d
