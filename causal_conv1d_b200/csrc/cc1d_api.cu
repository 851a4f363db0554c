// extern "C" entry points declared in include/cc1d.h: parameter validation (the checks the
// reference does with TORCH_CHECK in csrc/causal_conv1d.cpp) and hand-off to the launchers.
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <utility>

#include "cc1d.h"
#include "cc1d_kernels.h"
#include "cc1d_tma.cuh"

namespace cc1d {

int num_sms() {
    static std::mutex mu;
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            n = 148;
        }
        cached[dev] = n;
    }
    return cached[dev];
}

int resident_ctas_per_sm(const void *kernel, int threads, size_t dyn_smem) {
    static std::mutex mu;
    static std::map<std::pair<const void *, int>, int> cache;
    std::lock_guard<std::mutex> lock(mu);
    const auto key = std::make_pair(kernel, threads);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, dyn_smem) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        n = 2;
    }
    cache[key] = n;
    return n;
}

void allow_dynamic_smem(const void *kernel, size_t bytes) {
    static std::mutex mu;
    static std::map<std::pair<const void *, int>, size_t> granted;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
    std::lock_guard<std::mutex> lock(mu);
    size_t &have = granted[std::make_pair(kernel, dev)];
    if (have >= bytes) return;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) == cudaSuccess) have = bytes;
    else (void)cudaGetLastError();   // the launch that follows reports the failure
}

using TensorMapEncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                       const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled, resolved once through the runtime (no link-time dependency on libcuda)
static TensorMapEncodeFn tensor_map_encoder() {
    static TensorMapEncodeFn encode = nullptr;
    static bool looked_up = false;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!looked_up) {
        looked_up = true;
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess) {
            encode = reinterpret_cast<TensorMapEncodeFn>(fn);
        } else {
            (void)cudaGetLastError();
        }
    }
    return encode;
}

static CUtensorMapDataType tensor_map_dtype(int dtype) {
    return dtype == CC1D_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
           : dtype == CC1D_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
}

bool make_channel_last_tensor_map(CUtensorMap *map, int dtype, const void *base, int64_t dim, int64_t seqlen,
                                  int64_t batch, int64_t l_stride, int64_t batch_stride, int row_bytes) {
    const TensorMapEncodeFn encode = tensor_map_encoder();
    if (encode == nullptr) return false;
    const int es = elem_size(dtype);
    if (batch < 1) batch = 1;
    if (batch == 1 || batch_stride <= 0) batch_stride = l_stride * seqlen;   // unused extent: any legal stride
    const cuuint64_t dims[3] = {(cuuint64_t)dim, (cuuint64_t)seqlen, (cuuint64_t)batch};
    const cuuint64_t strides[2] = {(cuuint64_t)l_stride * es, (cuuint64_t)batch_stride * es};   // bytes, dims 1..2
    const cuuint32_t box[3] = {(cuuint32_t)(row_bytes / es), (cuuint32_t)kTmaRows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    if (strides[0] % 16 || strides[1] % 16 || strides[0] >= (1ull << 40) || strides[1] >= (1ull << 40)) return false;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return false;
    const CUresult rc = encode(map, tensor_map_dtype(dtype), 3, const_cast<void *>(base), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS;
}

bool make_channel_first_tensor_map(CUtensorMap *map, int dtype, const void *base, int64_t seqlen, int64_t dim,
                                   int64_t batch, int64_t c_stride, int64_t batch_stride, int box_tokens, int box_channels) {
    const TensorMapEncodeFn encode = tensor_map_encoder();
    if (encode == nullptr) return false;
    const int es = elem_size(dtype);
    if (batch < 1) batch = 1;
    if (batch == 1 || batch_stride <= 0) batch_stride = c_stride * dim;      // unused extent: any legal stride
    if (c_stride <= 0 || batch_stride <= 0) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)seqlen, (cuuint64_t)dim, (cuuint64_t)batch};
    const cuuint64_t strides[2] = {(cuuint64_t)c_stride * es, (cuuint64_t)batch_stride * es};   // bytes, dims 1..2
    const cuuint32_t box[3] = {(cuuint32_t)box_tokens, (cuuint32_t)box_channels, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    if ((box_tokens * es) % 16 || box_channels > 256) return false;
    if (strides[0] % 16 || strides[1] % 16 || strides[0] >= (1ull << 40) || strides[1] >= (1ull << 40)) return false;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return false;
    const CUresult rc = encode(map, tensor_map_dtype(dtype), 3, const_cast<void *>(base), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS;
}

namespace {

bool bad_dtype(int d) { return d != CC1D_F32 && d != CC1D_F16 && d != CC1D_BF16; }
bool elem_aligned(const void *p, int dtype) {
    return (reinterpret_cast<uintptr_t>(p) % (uintptr_t)elem_size(dtype)) == 0;
}

// Shared front checks; sets *channel_last by the reference's rule
// (csrc/causal_conv1d.cpp:175-181).
int check_conv_common(int itype, int wtype, int width, int64_t batch, int64_t dim, int64_t seqlen,
                      const void *x, int64_t x_bs, int64_t x_cs, int64_t x_ls, const void *weight,
                      bool *channel_last) {
    if (bad_dtype(itype) || bad_dtype(wtype)) return CC1D_ERR_DTYPE;
    if (width < 2 || width > 4) return CC1D_ERR_WIDTH;
    if (batch < 0 || dim < 0 || seqlen < 0) return CC1D_ERR_SHAPE;
    const bool empty = batch == 0 || dim == 0 || seqlen == 0;   // nothing to read: pointers may be NULL
    if ((!empty && x == nullptr) || (dim > 0 && weight == nullptr)) return CC1D_ERR_NULL;
    if (x_ls != 1 && x_cs != 1) return CC1D_ERR_STRIDE;
    if (!elem_aligned(x, itype) || !elem_aligned(weight, wtype)) return CC1D_ERR_ALIGN;
    *channel_last = x_cs == 1 && x_ls > 1;
    if (*channel_last) {
        if (dim % 8 != 0) return CC1D_ERR_CL_DIM;
        if (x_ls % 8 != 0 || (batch > 1 && x_bs % 8 != 0)) return CC1D_ERR_CL_STRIDE;
    }
    return CC1D_OK;
}

int check_same_layout(bool channel_last, int64_t bs, int64_t cs, int64_t ls, int64_t seqlen, int64_t dim,
                      int64_t batch) {
    if (channel_last) {
        if (cs != 1 && dim > 1) return CC1D_ERR_STRIDE;
        if ((seqlen > 1 && ls % 8 != 0) || (batch > 1 && bs % 8 != 0)) return CC1D_ERR_CL_STRIDE;
    } else {
        if (ls != 1 && seqlen > 1) return CC1D_ERR_STRIDE;
    }
    return CC1D_OK;
}

}  // namespace
}  // namespace cc1d

using namespace cc1d;

extern "C" {

int cc1d_abi_version(void) { return 4; }

size_t cc1d_peer_allreduce_buffer_bytes(int32_t world, int64_t count) { return peer_allreduce_buffer_bytes(world, count); }

int cc1d_peer_allreduce(const cc1d_peer_allreduce_params *p, cc1d_stream_t stream) {
    if (p == nullptr) return CC1D_ERR_NULL;
    if (p->world < 1 || p->world > CC1D_MAX_PEERS || p->rank < 0 || p->rank >= p->world || p->count < 0)
        return CC1D_ERR_SHAPE;
    if (p->count % 4 != 0) return CC1D_ERR_ALIGN;
    if (p->status == nullptr) return CC1D_ERR_NULL;
    if (p->count > 0 && (p->src == nullptr || p->dst == nullptr)) return CC1D_ERR_NULL;
    if (!is_aligned16(p->src) || !is_aligned16(p->dst)) return CC1D_ERR_ALIGN;
    for (int r = 0; r < p->world; ++r) {
        if (p->peer_base[r] == nullptr) return CC1D_ERR_NULL;
        if (!is_aligned16(p->peer_base[r])) return CC1D_ERR_ALIGN;
    }
    return launch_peer_allreduce(*p, reinterpret_cast<cudaStream_t>(stream));
}

int cc1d_wait_expired(void) {
    const int f = fwd_wait_expired(), b = bwd_wait_expired();
    if (f < 0 || b < 0) return -1;
    return (f != 0 ? 1 : 0) | (b != 0 ? 2 : 0);
}

const char *cc1d_status_str(int status) {
    switch (status) {
        case CC1D_OK: return "ok";
        case CC1D_ERR_NULL: return "a required pointer is NULL";
        case CC1D_ERR_DTYPE: return "unsupported dtype (need float32, float16 or bfloat16)";
        case CC1D_ERR_WIDTH: return "causal_conv1d only supports width between 2 and 4";
        case CC1D_ERR_SHAPE: return "invalid or inconsistent sizes";
        case CC1D_ERR_STRIDE: return "tensor must be contiguous along seqlen (channel-first) or along channels (channel-last), matching x";
        case CC1D_ERR_CL_DIM: return "causal_conv1d only supports channel dimension divisible by 8 for now";
        case CC1D_ERR_CL_STRIDE: return "causal_conv1d with channel last layout requires strides (stride(0) and stride(2)) to be multiples of 8";
        case CC1D_ERR_LAYOUT: return "seq_idx, initial_states and final_states are only supported for channel last layout";
        case CC1D_ERR_STATE_STRIDE: return "state tensors must have stride(1) == 1";
        case CC1D_ERR_STATE_LEN: return "conv_state_len must be >= width - 1";
        case CC1D_ERR_WORKSPACE: return "backward workspace missing or smaller than cc1d_bwd_workspace_bytes()";
        case CC1D_ERR_ALIGN: return "pointer or stride not aligned for the required access width";
        case CC1D_ERR_TOO_LARGE: return "problem size exceeds an internal index range";
        case CC1D_ERR_LAUNCH: return "CUDA kernel launch failed";
        case CC1D_ERR_SCRATCH_LIMIT: return "problem needs more scratch than cc1d_bwd_noalloc has built in (CC1D_NOALLOC_SCRATCH_BYTES); use cc1d_bwd with a caller workspace";
        case CC1D_ERR_SCRATCH_ADDRESS: return "cc1d_bwd_noalloc could not look up the address of its built-in scratch on this device";
        case CC1D_ERR_CAPTURE: return "the first cc1d_bwd_noalloc call on a device must be made outside stream capture";
        case CC1D_ERR_SEQ_IDX_STATES: return "seq_idx cannot be combined with initial_states / final_states (packed sequences with states: cc1d_prefill_varlen)";
        case CC1D_ERR_PHASE: return "cc1d_bwd_params.phase must be 0 (whole backward), 1 (main kernel) or 2 (finishing kernel)";
        default: return "unknown cc1d status";
    }
}

int cc1d_fwd(const cc1d_fwd_params *p, cc1d_stream_t stream) {
    if (p == nullptr) return CC1D_ERR_NULL;
    bool cl = false;
    int rc = check_conv_common(p->itype, p->wtype, p->width, p->batch, p->dim, p->seqlen, p->x,
                               p->x_batch_stride, p->x_c_stride, p->x_l_stride, p->weight, &cl);
    if (rc != CC1D_OK) return rc;
    if (p->batch == 0 || p->dim == 0 || p->seqlen == 0) return CC1D_OK;   // empty problem: nothing to write
    if (p->out == nullptr) return CC1D_ERR_NULL;
    if (!elem_aligned(p->out, p->itype)) return CC1D_ERR_ALIGN;
    rc = check_same_layout(cl, p->out_batch_stride, p->out_c_stride, p->out_l_stride, p->seqlen, p->dim, p->batch);
    if (rc != CC1D_OK) return rc;
    if (!cl && (p->seq_idx || p->initial_states || p->final_states)) return CC1D_ERR_LAYOUT;
    if (p->seq_idx && (p->initial_states || p->final_states)) return CC1D_ERR_SEQ_IDX_STATES;
    if (p->initial_states && p->initial_states_c_stride != 1 && p->dim > 1) return CC1D_ERR_STATE_STRIDE;
    if (p->final_states && p->final_states_c_stride != 1 && p->dim > 1) return CC1D_ERR_STATE_STRIDE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    // strides of extent-1 dimensions carry no information (PyTorch leaves them arbitrary)
    cc1d_fwd_params q = *p;
    if (q.batch <= 1) q.x_batch_stride = q.out_batch_stride = q.initial_states_batch_stride = q.final_states_batch_stride = 0;
    if (q.width == 2) q.initial_states_l_stride = q.final_states_l_stride = 0;
    return cl ? launch_fwd_channel_last(q, s) : launch_fwd_channel_first(q, s);
}

static int check_bwd(const cc1d_bwd_params *p, bool *cl) {
    if (p == nullptr) return CC1D_ERR_NULL;
    int rc = check_conv_common(p->itype, p->wtype, p->width, p->batch, p->dim, p->seqlen, p->x,
                               p->x_batch_stride, p->x_c_stride, p->x_l_stride, p->weight, cl);
    if (rc != CC1D_OK) return rc;
    const bool empty = p->batch == 0 || p->dim == 0 || p->seqlen == 0;   // only dweight/dbias get written (zeros)
    if ((!empty && (p->dout == nullptr || p->dx == nullptr)) || (p->dim > 0 && p->dweight == nullptr)) return CC1D_ERR_NULL;
    if ((p->bias == nullptr) != (p->dbias == nullptr)) return CC1D_ERR_NULL;
    if (!elem_aligned(p->dout, p->itype) || !elem_aligned(p->dx, p->itype) ||
        !elem_aligned(p->dweight, CC1D_F32) || !elem_aligned(p->dbias, CC1D_F32)) return CC1D_ERR_ALIGN;
    // dout normally has x's layout class; beside a channel-last x it may also be channel-first (seqlen
    // stride 1, 16-bit types, 16-byte aligned rows): the backward then reads it in place
    const bool dout_cf = *cl && p->seqlen > 1 && p->dim > 1 && p->dout_l_stride == 1 && p->dout_c_stride != 1;
    if (dout_cf) {
        if (p->itype == CC1D_F32 || p->dout_c_stride % 8 != 0 || (p->batch > 1 && p->dout_batch_stride % 8 != 0))
            return CC1D_ERR_STRIDE;
    } else {
        rc = check_same_layout(*cl, p->dout_batch_stride, p->dout_c_stride, p->dout_l_stride, p->seqlen, p->dim, p->batch);
        if (rc != CC1D_OK) return rc;
    }
    rc = check_same_layout(*cl, p->dx_batch_stride, p->dx_c_stride, p->dx_l_stride, p->seqlen, p->dim, p->batch);
    if (rc != CC1D_OK) return rc;
    if (!*cl && (p->seq_idx || p->initial_states || p->dfinal_states || p->dinitial_states)) return CC1D_ERR_LAYOUT;
    if (p->seq_idx && (p->initial_states || p->dfinal_states || p->dinitial_states)) return CC1D_ERR_SEQ_IDX_STATES;
    if (p->phase < 0 || p->phase > 2) return CC1D_ERR_PHASE;
    if (p->initial_states && p->initial_states_c_stride != 1 && p->dim > 1) return CC1D_ERR_STATE_STRIDE;
    if (p->dinitial_states && p->dinitial_states_c_stride != 1 && p->dim > 1) return CC1D_ERR_STATE_STRIDE;
    if (p->peers != nullptr) {
        const cc1d_peer_group *g = p->peers;
        if (g->world < 1 || g->world > CC1D_MAX_PEERS || g->rank < 0 || g->rank >= g->world) return CC1D_ERR_SHAPE;
        if (g->capacity < p->dim * (int64_t)(p->width + 1)) return CC1D_ERR_SHAPE;
        if (g->status == nullptr) return CC1D_ERR_NULL;
        for (int r = 0; r < g->world; ++r) {
            if (g->peer_base[r] == nullptr) return CC1D_ERR_NULL;
            if (!is_aligned16(g->peer_base[r])) return CC1D_ERR_ALIGN;
        }
    }
    return CC1D_OK;
}

size_t cc1d_bwd_workspace_bytes(const cc1d_bwd_params *p) {
    if (p == nullptr || bad_dtype(p->itype) || p->width < 2 || p->width > 4 || p->batch < 0 || p->dim < 0 ||
        p->seqlen < 0) return 0;
    const bool cl = p->x_c_stride == 1 && p->x_l_stride > 1;
    const size_t n = cl ? bwd_workspace_bytes_channel_last(*p) : bwd_workspace_bytes_channel_first(*p);
    return n < 16 ? 16 : n;   // never 0 for a valid problem, so callers can always allocate
}

// Checked parameters -> launcher.  The launchers test the workspace against the partial rows of
// the tiling they actually pick (CC1D_ERR_WORKSPACE when it is too small).
static int run_bwd(const cc1d_bwd_params *p, bool cl, cc1d_stream_t stream) {
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    cc1d_bwd_params q = *p;
    if (q.batch <= 1) {
        q.x_batch_stride = q.dout_batch_stride = q.dx_batch_stride = 0;
        q.initial_states_batch_stride = q.dfinal_states_batch_stride = q.dinitial_states_batch_stride = 0;
    }
    if (q.width == 2) q.initial_states_l_stride = q.dfinal_states_l_stride = q.dinitial_states_l_stride = 0;
    return cl ? launch_bwd_channel_last(q, s) : launch_bwd_channel_first(q, s);
}

int cc1d_bwd(const cc1d_bwd_params *p, cc1d_stream_t stream) {
    bool cl = false;
    const int rc = check_bwd(p, &cl);
    if (rc != CC1D_OK) return rc;
    if (p->workspace == nullptr || p->workspace_bytes < cc1d_bwd_workspace_bytes(p)) return CC1D_ERR_WORKSPACE;
    return run_bwd(p, cl, stream);
}

}  // extern "C"

// Scratch of cc1d_bwd_noalloc: part of the library image, so no allocation is ever needed.
// In host code the name below is only a host-side stand-in for the symbol, not a device
// address; the address a kernel can use comes from cudaGetSymbolAddress, looked up once per
// device (with that device current) and cached.
static __device__ __align__(256) unsigned char g_noalloc_scratch[CC1D_NOALLOC_SCRATCH_BYTES];

namespace {
std::mutex g_scratch_mu;
void *g_scratch_ptr[64] = {nullptr};

// Device address of g_noalloc_scratch on the current device.  The first call per device does the
// lookup, which may load the library's device code: not something to do while `stream` is being
// captured, so that case is refused instead.
int noalloc_scratch_address(cudaStream_t stream, void **out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return CC1D_ERR_SCRATCH_ADDRESS;
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    if (g_scratch_ptr[dev] == nullptr) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) {
            (void)cudaGetLastError();
            return CC1D_ERR_SCRATCH_ADDRESS;
        }
        if (cap != cudaStreamCaptureStatusNone) return CC1D_ERR_CAPTURE;
        void *ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || ptr == nullptr) {
            (void)cudaGetLastError();
            return CC1D_ERR_SCRATCH_ADDRESS;
        }
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return CC1D_OK;
}
}  // namespace

extern "C" {

int cc1d_bwd_noalloc(const cc1d_bwd_params *p, cc1d_stream_t stream) {
    bool cl = false;
    const int rc = check_bwd(p, &cl);
    if (rc != CC1D_OK) return rc;
    void *scratch = nullptr;   // first call per device: one symbol lookup
    const int arc = noalloc_scratch_address(reinterpret_cast<cudaStream_t>(stream), &scratch);
    if (arc != CC1D_OK) return arc;
    cc1d_bwd_params q = *p;
    q.workspace = scratch;
    q.workspace_bytes = CC1D_NOALLOC_SCRATCH_BYTES;
    // the launcher sizes the partial rows for the tiling these pointers select and launches
    // nothing when they do not fit
    const int lrc = run_bwd(&q, cl, stream);
    return lrc == CC1D_ERR_WORKSPACE ? CC1D_ERR_SCRATCH_LIMIT : lrc;
}

int cc1d_update(const cc1d_update_params *p, cc1d_stream_t stream) {
    if (p == nullptr) return CC1D_ERR_NULL;
    if (bad_dtype(p->itype) || bad_dtype(p->wtype)) return CC1D_ERR_DTYPE;
    if (p->width < 2 || p->width > 4) return CC1D_ERR_WIDTH;
    if (p->batch < 0 || p->dim < 0 || p->seqlen < 0 || p->conv_state_len < 0) return CC1D_ERR_SHAPE;
    if (p->conv_state_len < p->width - 1) return CC1D_ERR_STATE_LEN;
    if (p->batch == 0 || p->dim == 0 || p->seqlen == 0) return CC1D_OK;   // empty problem
    if (p->x == nullptr || p->weight == nullptr || p->out == nullptr || p->conv_state == nullptr) return CC1D_ERR_NULL;
    if (!elem_aligned(p->x, p->itype) || !elem_aligned(p->out, p->itype) || !elem_aligned(p->conv_state, p->itype) ||
        !elem_aligned(p->weight, p->wtype)) return CC1D_ERR_ALIGN;
    return launch_update(*p, reinterpret_cast<cudaStream_t>(stream));
}

int cc1d_varlen_states(const cc1d_varlen_states_params *p, cc1d_stream_t stream) {
    if (p == nullptr) return CC1D_ERR_NULL;
    if (bad_dtype(p->itype)) return CC1D_ERR_DTYPE;
    if (p->total_tokens < 0 || p->dim < 0 || p->batch < 0 || p->state_len < 0) return CC1D_ERR_SHAPE;
    if (p->batch == 0 || p->dim == 0 || p->state_len == 0) return CC1D_OK;
    if ((p->x == nullptr && p->total_tokens > 0) || p->cu_seqlens == nullptr || p->states == nullptr) return CC1D_ERR_NULL;
    if (!elem_aligned(p->x, p->itype) || !elem_aligned(p->states, p->itype)) return CC1D_ERR_ALIGN;
    return launch_varlen_states(*p, reinterpret_cast<cudaStream_t>(stream));
}

int cc1d_seq_idx_from_cu_seqlens(const int32_t *cu_seqlens, int64_t nseq, int64_t total_tokens, int32_t *seq_idx,
                                 cc1d_stream_t stream) {
    if (nseq < 0 || total_tokens < 0) return CC1D_ERR_SHAPE;
    if (total_tokens == 0) return CC1D_OK;
    if (cu_seqlens == nullptr || seq_idx == nullptr) return CC1D_ERR_NULL;
    return launch_seq_idx(cu_seqlens, nseq, total_tokens, seq_idx, reinterpret_cast<cudaStream_t>(stream));
}

int cc1d_prefill_varlen(const cc1d_prefill_varlen_params *p, cc1d_stream_t stream) {
    if (p == nullptr) return CC1D_ERR_NULL;
    if (p->nseq < 0 || p->state_len < 0 || p->total_tokens < 0 || p->dim < 0) return CC1D_ERR_SHAPE;
    if (bad_dtype(p->itype) || bad_dtype(p->wtype)) return CC1D_ERR_DTYPE;
    if (p->width < 2 || p->width > 4) return CC1D_ERR_WIDTH;
    if (p->dim % 8 != 0) return CC1D_ERR_CL_DIM;
    // cu_seqlens and seq_idx are int32, and the kernels index tokens with 32-bit integers
    if (p->total_tokens >= (1ll << 31) - 4096) return CC1D_ERR_TOO_LARGE;
    const bool states = p->initial_states != nullptr || p->final_states != nullptr;
    if (states && p->state_len < p->width - 1) return CC1D_ERR_STATE_LEN;
    if (p->dim == 0) return CC1D_OK;
    if (p->nseq > 0 && p->cu_seqlens == nullptr) return CC1D_ERR_NULL;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int C = vec_elems(p->itype);

    if (p->total_tokens > 0 && (p->seq_idx == nullptr || p->x == nullptr || p->out == nullptr)) return CC1D_ERR_NULL;
    if (p->total_tokens > 0 && (p->x_l_stride <= 1 || p->out_l_stride <= 1)) return CC1D_ERR_STRIDE;
    if (states && p->nseq > 0) {
        // the boundary kernel moves 16-byte channel vectors
        if (p->total_tokens > 0 && (!is_aligned16(p->x) || !is_aligned16(p->out) || p->x_l_stride % C || p->out_l_stride % C))
            return CC1D_ERR_ALIGN;
        if (p->initial_states != nullptr && (!is_aligned16(p->initial_states) || p->initial_states_batch_stride % C ||
                                             (p->state_len > 1 && p->initial_states_l_stride % C)))
            return CC1D_ERR_ALIGN;
        if (p->final_states != nullptr && (!is_aligned16(p->final_states) || p->final_states_batch_stride % C ||
                                           (p->state_len > 1 && p->final_states_l_stride % C)))
            return CC1D_ERR_ALIGN;
    }
    if (p->total_tokens > 0) {
        // the masked channel-last forward over the whole pack, as one batch entry
        cc1d_fwd_params f = {};
        f.itype = p->itype; f.wtype = p->wtype; f.width = p->width; f.silu = p->silu;
        f.batch = 1; f.dim = p->dim; f.seqlen = p->total_tokens;
        f.x = p->x; f.x_c_stride = 1; f.x_l_stride = p->x_l_stride;
        f.weight = p->weight; f.weight_c_stride = p->weight_c_stride; f.weight_width_stride = p->weight_width_stride;
        f.bias = p->bias;
        f.out = p->out; f.out_c_stride = 1; f.out_l_stride = p->out_l_stride;
        f.seq_idx = p->seq_idx;
        const int rc = cc1d_fwd(&f, stream);
        if (rc != CC1D_OK) return rc;
    }
    if (!states || p->nseq == 0) return CC1D_OK;
    return launch_prefill_boundary(*p, s);
}

}  // extern "C"
