// Packed variable-length prefill with per-sequence conv states (sm_100a).
//
// The bulk of the work is the channel-last forward with seq_idx masking (cc1d_fwd.cu); this
// file adds the two small kernels around it:
//   seq_idx_kernel          seq_idx[t] from cu_seqlens (binary search per token);
//   prefill_boundary_kernel per (sequence, 16-byte channel vector): recompute the first width-1
//                           outputs of a sequence that continues from a stored state (the
//                           masked forward treated its left context as zeros) and write the
//                           sequence's final state, last state_len entries of [prefix | x_s].
// The boundary kernel repeats the forward's arithmetic operation for operation (same tap
// order, same SiLU form), so a token it rewrites gets the bits the forward would have
// produced had it seen the prefix.
#include "cc1d_common.cuh"
#include "cc1d_kernels.h"

namespace cc1d {

__global__ void __launch_bounds__(256) seq_idx_kernel(const int32_t *__restrict__ cu, int nseq, int64_t total,
                                                      int32_t *__restrict__ seq_idx) {
    pdl_wait();
    const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (t >= total) return;
    // largest s with cu[s] <= t; empty sequences (cu[s] == cu[s+1]) are skipped by taking the last
    int lo = 0, hi = nseq;   // invariant: cu[lo] <= t, and (hi == nseq or cu[hi] > t)
    if (nseq == 0 || t >= cu[nseq]) { seq_idx[t] = -1; return; }
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (cu[mid] <= t) lo = mid; else hi = mid;
    }
    seq_idx[t] = lo;
}

struct PrefillArgs {
    const void *x;
    void *out;
    const void *weight;
    const void *bias;
    const int32_t *cu;
    const int32_t *idx;
    const uint8_t *has;
    const void *init;
    void *fin;
    int64_t x_ls, o_ls, w_cs, w_ws, i_bs, i_ls, f_bs, f_ls;
    int wtype;
    int S;
    uint32_t ncols;     // 16-byte channel vectors per token
    uint32_t ncolblk;   // CTAs along channels
};

template <typename T, int W, bool kSilu>
__global__ void __launch_bounds__(128) prefill_boundary_kernel(const PrefillArgs a) {
    pdl_wait();
    constexpr int C = Elem<T>::kVec;
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
    const uint32_t cb = blockIdx.x % a.ncolblk;
    const int s = (int)(blockIdx.x / a.ncolblk);
    const uint32_t col = cb * 128 + threadIdx.x;
    if (col >= a.ncols) return;
    const int64_t beg = a.cu[s], end = a.cu[s + 1];
    const int64_t len = end - beg;
    const int64_t row = a.idx != nullptr ? (int64_t)a.idx[s] : (int64_t)s;
    const bool prefixed = a.init != nullptr && row >= 0 && (a.has == nullptr || a.has[s] != 0);
    const T *xcol = reinterpret_cast<const T *>(a.x) + (int64_t)col * C;
    const T *icol = prefixed ? reinterpret_cast<const T *>(a.init) + row * a.i_bs + (int64_t)col * C : nullptr;
    const int S = a.S;

    // Everything the thread reads is requested before anything is written, so that the kernel is
    // one round trip to memory deep: left context, the first width-1 tokens, the taps, and the
    // sources of the first kChunk state slots.
    constexpr int kChunk = 4;
    const bool redo = prefixed && len > 0;
    const bool store_state = a.fin != nullptr && row >= 0;
    uint4 ctx[W - 1], tok[W - 1], src[kChunk];
    #pragma unroll
    for (int k = 0; k < W - 1; ++k) {
        ctx[k] = tok[k] = make_uint4(0, 0, 0, 0);
        if (redo) ctx[k] = ld_cached(icol + (int64_t)(S - (W - 1) + k) * a.i_ls);
        if (redo && k < len) tok[k] = ld_cached(xcol + (beg + k) * a.x_ls);
    }
    // state slot k <- element len + k of [prefix (S entries) | x_s (len entries)]
    auto state_source = [&](int k) {
        const int64_t e = len + k;
        if (k >= S || !store_state) return make_uint4(0, 0, 0, 0);
        if (e >= S) return ld_cached(xcol + (beg + e - S) * a.x_ls);
        if (prefixed) return ld_cached(icol + e * a.i_ls);
        return make_uint4(0, 0, 0, 0);
    };
    #pragma unroll
    for (int k = 0; k < kChunk; ++k) src[k] = state_source(k);

    if (redo) {
        float win[W - 1][C];
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) unpack<T>(ctx[k], win[k]);
        float wv[W][C], bv[C];
        load_taps<W, C>(wv, bv, a.weight, a.w_cs, a.w_ws, a.bias, a.wtype, (int64_t)col * C, kTanh ? 0.5f : 1.f);
        T *ocol = reinterpret_cast<T *>(a.out) + (int64_t)col * C;
        #pragma unroll
        for (int j = 0; j < W - 1; ++j) {
            if (j < len) {
                float cur[C], o[C];
                unpack<T>(tok[j], cur);
                #pragma unroll
                for (int c = 0; c < C; ++c) {
                    float acc = bv[c];
                    #pragma unroll
                    for (int k = 0; k < W - 1; ++k) acc = fmaf(wv[k][c], win[k][c], acc);
                    acc = fmaf(wv[W - 1][c], cur[c], acc);
                    if (kSilu) acc = kTanh ? silu_half_arg(acc) : silu_f(acc);
                    o[c] = acc;
                }
                *reinterpret_cast<uint4 *>(ocol + (beg + j) * a.o_ls) = pack<T>(o);
                #pragma unroll
                for (int k = 0; k < W - 2; ++k) {
                    #pragma unroll
                    for (int c = 0; c < C; ++c) win[k][c] = win[k + 1][c];
                }
                #pragma unroll
                for (int c = 0; c < C; ++c) win[W - 2][c] = cur[c];
            }
        }
    }

    // Final state, kChunk slots at a time: sources first, then the stores.  Slot k's source is
    // never a slot written earlier (len + k >= k, and chunks go upwards), so the update may run
    // in place on the row the prefix came from.
    if (store_state) {
        T *fcol = reinterpret_cast<T *>(a.fin) + row * a.f_bs + (int64_t)col * C;
        for (int k0 = 0; k0 < S; k0 += kChunk) {
            if (k0 > 0) {
                #pragma unroll
                for (int k = 0; k < kChunk; ++k) src[k] = state_source(k0 + k);
            }
            #pragma unroll
            for (int k = 0; k < kChunk; ++k) {
                if (k0 + k < S) *reinterpret_cast<uint4 *>(fcol + (int64_t)(k0 + k) * a.f_ls) = src[k];
            }
        }
    }
}

int launch_seq_idx(const int32_t *cu, int64_t nseq, int64_t total, int32_t *seq_idx, cudaStream_t stream) {
    if (total == 0) return CC1D_OK;
    const uint64_t ctas = ((uint64_t)total + 255) / 256;
    if (ctas >= (1ull << 31) || nseq >= (1ll << 30)) return CC1D_ERR_TOO_LARGE;
    launch_k(seq_idx_kernel, dim3((unsigned)ctas), dim3(256), 0, stream, cu, (int)nseq, total, seq_idx);
    return check_launch();
}

int launch_prefill_boundary(const cc1d_prefill_varlen_params &p, cudaStream_t stream) {
    if (p.nseq == 0 || p.dim == 0) return CC1D_OK;
    if (p.initial_states == nullptr && p.final_states == nullptr) return CC1D_OK;
    const int C = vec_elems(p.itype);
    PrefillArgs a;
    a.x = p.x; a.out = p.out; a.weight = p.weight; a.bias = p.bias;
    a.cu = p.cu_seqlens; a.idx = p.state_indices; a.has = p.has_initial_state;
    a.init = p.initial_states; a.fin = p.final_states;
    a.x_ls = p.x_l_stride; a.o_ls = p.out_l_stride; a.w_cs = p.weight_c_stride; a.w_ws = p.weight_width_stride;
    a.i_bs = p.initial_states_batch_stride; a.i_ls = p.initial_states_l_stride;
    a.f_bs = p.final_states_batch_stride; a.f_ls = p.final_states_l_stride;
    a.wtype = p.wtype; a.S = (int)p.state_len;
    a.ncols = (uint32_t)(p.dim / C);
    a.ncolblk = (a.ncols + 127) / 128;
    const uint64_t ctas = (uint64_t)a.ncolblk * (uint64_t)p.nseq;
    if (ctas >= (1ull << 31)) return CC1D_ERR_TOO_LARGE;
    CC1D_DISPATCH_ITYPE(p.itype, CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu, {
        launch_k(prefill_boundary_kernel<T, W, kSilu>, dim3((unsigned)ctas), dim3(128), 0, stream, a);
    });););
    return check_launch();
}

}  // namespace cc1d
