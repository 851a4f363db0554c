// Variable-length "last tokens -> conv state" gather (sm_100a).  Replaces the Triton kernel
// _causal_conv1d_varlen_states (causal_conv1d/causal_conv1d_varlen.py:8-32 of the reference):
//   n = min(state_len, cu[b+1] - cu[b]);  states[b, :, state_len-n:] = x[cu[b+1]-n : cu[b+1], :].T
// and zeros in front.  A pure copy: bit-exact by construction.
#include "cc1d_common.cuh"
#include "cc1d_kernels.h"

namespace cc1d {

struct VarlenArgs {
    const void *x;
    const void *cu;
    void *states;
    int64_t x_ls, x_cs, s_bs, s_cs, s_ls;
    int64_t dim, state_len;
    int cu_is64;
    uint32_t ncols;    // vector path: 16-byte vectors per token; scalar path: dim
    uint32_t ncolblk;  // CTAs along channels
};

__device__ __forceinline__ int64_t load_cu(const void *cu, int64_t i, int is64) {
    return is64 ? reinterpret_cast<const int64_t *>(cu)[i] : (int64_t)reinterpret_cast<const int32_t *>(cu)[i];
}

// kVec: thread copies one 16-byte vector of channels (x and states both channel-contiguous);
// otherwise one element with arbitrary strides.  Flat grid over (batch entry, state slot, column block).
template <typename T, bool kVec>
__global__ void __launch_bounds__(128) varlen_states_kernel(const VarlenArgs a) {
    pdl_wait();
    constexpr int C = kVec ? Elem<T>::kVec : 1;
    const uint32_t cb = blockIdx.x % a.ncolblk;
    const uint32_t rest = blockIdx.x / a.ncolblk;
    const int64_t k = rest % (uint32_t)a.state_len;    // state slot
    const int64_t b = rest / (uint32_t)a.state_len;
    const uint32_t col = cb * 128 + threadIdx.x;
    if (col >= a.ncols) return;
    const int64_t end = load_cu(a.cu, b + 1, a.cu_is64);
    const int64_t beg = load_cu(a.cu, b, a.cu_is64);
    const int64_t tok = end - a.state_len + k;           // token feeding slot k
    const bool live = tok >= beg && tok >= 0;
    T *dst = reinterpret_cast<T *>(a.states) + b * a.s_bs + k * a.s_ls + (int64_t)col * C * (kVec ? 1 : a.s_cs);
    if (kVec) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (live) v = ld_stream(reinterpret_cast<const T *>(a.x) + tok * a.x_ls + (int64_t)col * C);
        *reinterpret_cast<uint4 *>(dst) = v;
    } else {
        T v = Elem<T>::from_f(0.f);
        if (live) v = reinterpret_cast<const T *>(a.x)[tok * a.x_ls + (int64_t)col * a.x_cs];
        *dst = v;
    }
}

int launch_varlen_states(const cc1d_varlen_states_params &p, cudaStream_t stream) {
    if (p.batch == 0 || p.dim == 0 || p.state_len == 0) return CC1D_OK;
    const int C = vec_elems(p.itype);
    VarlenArgs a;
    a.x = p.x; a.cu = p.cu_seqlens; a.states = p.states;
    a.x_ls = p.x_l_stride; a.x_cs = p.x_c_stride;
    a.s_bs = p.states_batch_stride; a.s_cs = p.states_c_stride; a.s_ls = p.states_l_stride;
    a.dim = p.dim; a.state_len = p.state_len; a.cu_is64 = p.cu_seqlens_is_int64;
    const bool vec = p.dim % C == 0 && p.x_c_stride == 1 && p.states_c_stride == 1 && is_aligned16(p.x) &&
                     is_aligned16(p.states) && p.x_l_stride % C == 0 && p.states_batch_stride % C == 0 &&
                     p.states_l_stride % C == 0;
    a.ncols = (uint32_t)(vec ? p.dim / C : p.dim);
    a.ncolblk = (a.ncols + 127) / 128;
    if (p.state_len >= (1ll << 31) || p.batch >= (1ll << 31)) return CC1D_ERR_TOO_LARGE;
    const uint64_t gx = (uint64_t)a.ncolblk * (uint64_t)p.state_len * (uint64_t)p.batch;
    if (gx >= (1ull << 31)) return CC1D_ERR_TOO_LARGE;
    const dim3 grid((unsigned)gx);
    CC1D_DISPATCH_ITYPE(p.itype, CC1D_DISPATCH_BOOL(vec, kVec, {
        launch_k(varlen_states_kernel<T, kVec>, dim3(grid), dim3(128), 0, stream, a);
    }););
    return check_launch();
}

}  // namespace cc1d
