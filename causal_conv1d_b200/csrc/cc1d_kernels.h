// Internal launch functions behind the C ABI (cc1d_api.cu validates, these dispatch on
// dtype / width / flags and launch).  All return a cc1d_status.
#pragma once

#include <cuda_runtime.h>

#include <utility>

#include "cc1d.h"

// Compile-time tunables (overridable with -D for experiments).
#ifndef CC1D_CF_KVECS
#define CC1D_CF_KVECS 4          // 16-byte vectors per lane per group, channel-first kernels
#endif
#ifndef CC1D_CF_FWD_PERSISTENT
#define CC1D_CF_FWD_PERSISTENT 0   // 1: grid = resident CTAs with a grid-stride loop; 0: one warp unit per warp
#endif
#ifndef CC1D_CF_BWD_PERSISTENT
#define CC1D_CF_BWD_PERSISTENT 2   // 2: persistent only for 16-bit I/O (issue-bound), one unit per warp for fp32
#endif

namespace cc1d {

constexpr int kCfVecs = CC1D_CF_KVECS;
constexpr int kCfGroupVecs = 32 * kCfVecs;

// Number of SMs of the current device (cached per device; 148 on B200).
int num_sms();

inline bool is_aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int elem_size(int dtype) { return dtype == CC1D_F32 ? 4 : 2; }
inline int vec_elems(int dtype) { return 16 / elem_size(dtype); }

uint64_t groups_per_unit(uint64_t rows, uint64_t groups_per_row);
int launch_fwd_channel_first(const cc1d_fwd_params &p, cudaStream_t stream);
int launch_fwd_channel_last(const cc1d_fwd_params &p, cudaStream_t stream);

size_t bwd_workspace_bytes_channel_first(const cc1d_bwd_params &p);
size_t bwd_workspace_bytes_channel_last(const cc1d_bwd_params &p);
int launch_bwd_channel_first(const cc1d_bwd_params &p, cudaStream_t stream);
int launch_bwd_channel_last(const cc1d_bwd_params &p, cudaStream_t stream);

size_t peer_allreduce_buffer_bytes(int world, int64_t count);
int launch_peer_allreduce(const cc1d_peer_allreduce_params &p, cudaStream_t stream);
int fwd_wait_expired();   // bounded-wait flags of the TMA kernels, per translation unit (synchronise)
int bwd_wait_expired();
int launch_update(const cc1d_update_params &p, cudaStream_t stream);
int launch_varlen_states(const cc1d_varlen_states_params &p, cudaStream_t stream);
int launch_seq_idx(const int32_t *cu, int64_t nseq, int64_t total, int32_t *seq_idx, cudaStream_t stream);
int launch_prefill_boundary(const cc1d_prefill_varlen_params &p, cudaStream_t stream);

// Resident CTAs per SM of a kernel (occupancy query, cached per kernel and block size):
// persistent grid-stride kernels launch exactly sms * this many CTAs, so that no partial
// second wave forms.
int resident_ctas_per_sm(const void *kernel, int threads, size_t dyn_smem);

// Opt a kernel in to `bytes` of dynamic shared memory (> 48 KB needs it).  The attribute
// belongs to the device's context, so it is set once per (kernel, device), not once per process.
void allow_dynamic_smem(const void *kernel, size_t bytes);

template <typename K>
inline unsigned persistent_grid(K kernel, int threads, uint64_t ctas_wanted, bool persistent = true) {
    if (!persistent) return (unsigned)ctas_wanted;
    const uint64_t cap = (uint64_t)num_sms() * (uint64_t)resident_ctas_per_sm(reinterpret_cast<const void *>(kernel), threads, 0);
    return (unsigned)(ctas_wanted < cap ? ctas_wanted : cap);
}

// Every kernel of this library is launched with programmatic stream serialisation: the next
// kernel of the stream may be scheduled onto SMs that the previous one has vacated while its
// last CTAs still run.  Each kernel starts with griddepcontrol.wait (pdl_wait() in
// cc1d_common.cuh), which returns only when the kernels before it in the stream have
// completed and their writes are visible, so stream order is unchanged for every memory access;
// what overlaps is launch latency, CTA scheduling and the tail of the previous kernel.
#ifndef CC1D_PDL
#define CC1D_PDL 1
#endif
// Status of the launches made since the last check_launch() on this host thread: launch_k keeps
// the first cudaError_t that cudaLaunchKernelEx itself returned.  Nothing here calls
// cudaGetLastError() on the success path, so an earlier, unrelated error that the host
// application has not collected yet is neither reported as ours nor wiped.
inline cudaError_t &pending_launch_error() {
    static thread_local cudaError_t err = cudaSuccess;
    return err;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = CC1D_PDL ? 1 : 0;
    const cudaError_t rc = cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
    if (rc != cudaSuccess && pending_launch_error() == cudaSuccess) pending_launch_error() = rc;
    return rc;
}

// CC1D_ERR_LAUNCH when a launch_k since the previous call failed; the failed launch's own
// (non-sticky) error is cleared so that it is reported once.
inline int check_launch() {
    cudaError_t &err = pending_launch_error();
    if (err == cudaSuccess) return CC1D_OK;
    err = cudaSuccess;
    (void)cudaGetLastError();
    return CC1D_ERR_LAUNCH;
}

}  // namespace cc1d

// Dispatch helpers: run `...` (a generic lambda body) with T / W bound as types / constants.
#define CC1D_DISPATCH_ITYPE(itype, ...)                                         \
    do {                                                                        \
        if ((itype) == CC1D_F32) { using T = float; __VA_ARGS__ }               \
        else if ((itype) == CC1D_F16) { using T = __half; __VA_ARGS__ }         \
        else { using T = __nv_bfloat16; __VA_ARGS__ }                           \
    } while (0)

#define CC1D_DISPATCH_WIDTH(width, ...)                                         \
    do {                                                                        \
        if ((width) == 2) { constexpr int W = 2; __VA_ARGS__ }                  \
        else if ((width) == 3) { constexpr int W = 3; __VA_ARGS__ }             \
        else { constexpr int W = 4; __VA_ARGS__ }                               \
    } while (0)

#define CC1D_DISPATCH_BOOL(cond, NAME, ...)                                     \
    do {                                                                        \
        if (cond) { constexpr bool NAME = true; __VA_ARGS__ }                   \
        else { constexpr bool NAME = false; __VA_ARGS__ }                       \
    } while (0)
