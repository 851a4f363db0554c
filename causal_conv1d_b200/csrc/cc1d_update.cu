// Decode-step state update kernels (sm_100a).  Replaces causal_conv1d_update_kernel
// (csrc/causal_conv1d_update.cu:23-114 of the reference).
//
// Vector path (x, out and conv_state all have channel stride 1): a thread owns one 16-byte
// vector of channels of one batch entry; a warp touches 512 contiguous bytes per state row /
// token.  The width-1 window is read once, the state shift is done in registers when
// state_len == width-1 and as row copies otherwise.
//
// Generic path: any strides, one (batch, channel) pair per thread, scalar accesses.
#include "cc1d_common.cuh"
#include "cc1d_kernels.h"

namespace cc1d {

struct UpdArgs {
    const void *x;
    void *out;
    void *state;
    const void *weight;
    const void *bias;
    const int32_t *cache_seqlens;
    const int32_t *indices;
    int64_t x_bs, x_cs, x_ls, o_bs, o_cs, o_ls, s_bs, s_cs, s_ls, w_cs, w_ws;
    int64_t dim;
    int32_t batch, seqlen, state_len;
    int wtype;
    uint32_t ncols, ncolblk;
};

constexpr int kUpdRows = 4;     // batch entries per CTA (threadIdx.y)
constexpr int kUpdUnroll = 4;   // tokens loaded together

template <typename T, int W, bool kSilu, bool kCirc>
__global__ void __launch_bounds__(32 * kUpdRows) update_vec_kernel(const UpdArgs a) {
    constexpr int C = Elem<T>::kVec;
    __shared__ __align__(16) float s_w[(W + 1) * 32 * C];

    const uint32_t cb = blockIdx.x % a.ncolblk;
    const uint32_t bg = blockIdx.x / a.ncolblk;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int32_t b = (int32_t)bg * kUpdRows + ty;

    // the state row index is the head of the dependent-load chain: fetch it first
    int32_t coord = -1, cs = 0;
    if (b < a.batch) {
        coord = a.indices != nullptr ? a.indices[b] : b;
        if (kCirc) cs = a.cache_seqlens[b];
    }
    stage_weights<W>(s_w, 32 * C, (int64_t)cb * 32 * C, a.dim, a.weight, a.w_cs, a.w_ws, a.bias,
                     a.wtype, threadIdx.x, 32 * kUpdRows);
    __syncthreads();

    const uint32_t col = cb * 32 + tx;
    if (col >= a.ncols || b >= a.batch) return;
    const T *__restrict__ xp = reinterpret_cast<const T *>(a.x) + b * a.x_bs + (int64_t)col * C;
    T *__restrict__ op = reinterpret_cast<T *>(a.out) + b * a.o_bs + (int64_t)col * C;
    const int L = a.seqlen, S = a.state_len;

    if (coord < 0) {  // padded entry: zero output, state untouched
        for (int i = 0; i < L; ++i) st_stream(op + i * a.o_ls, make_uint4(0, 0, 0, 0));
        return;
    }
    T *sp = reinterpret_cast<T *>(a.state) + coord * a.s_bs + (int64_t)col * C;

    // window rows (the width-1 entries that precede x)
    int widx[W - 1];
    int wr = 0;  // circular: first row x is written to
    if (kCirc) {
        wr = cs % S;  // cache_seqlens >= 0 by contract; a negative value is folded below
        if (wr < 0) wr += S;
        int r = wr - (W - 1);
        if (r < 0) r += S;   // state_len >= width-1
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) { widx[k] = r; r = r + 1 >= S ? r + 1 - S : r + 1; }
    } else {
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) widx[k] = S - (W - 1) + k;
    }
    uint4 wraw[W - 1];
    #pragma unroll
    for (int k = 0; k < W - 1; ++k) wraw[k] = ld_cached(sp + widx[k] * a.s_ls);

    float wv[W][C], bv[C];
    #pragma unroll
    for (int k = 0; k < W; ++k) {
        #pragma unroll
        for (int c = 0; c < C; ++c) wv[k][c] = s_w[k * 32 * C + tx * C + c];
    }
    #pragma unroll
    for (int c = 0; c < C; ++c) bv[c] = s_w[W * 32 * C + tx * C + c];

    // linear mode with spare rows: shift the surviving rows down by L (ascending, in place)
    const bool in_regs = !kCirc && S == W - 1;  // new state == final window
    if (!kCirc && !in_regs) {
        #pragma unroll 4
        for (int i = 0; i < S - L; ++i) {
            const uint4 v = ld_cached(sp + (i + L) * a.s_ls);
            *reinterpret_cast<uint4 *>(sp + i * a.s_ls) = v;
        }
    }

    float win[W - 1][C];
    #pragma unroll
    for (int k = 0; k < W - 1; ++k) unpack<T>(wraw[k], win[k]);

    for (int t = 0; t < L; t += kUpdUnroll) {
        uint4 raw[kUpdUnroll];
        #pragma unroll
        for (int u = 0; u < kUpdUnroll; ++u) {
            raw[u] = make_uint4(0, 0, 0, 0);
            if (t + u < L) raw[u] = ld_stream(xp + (t + u) * a.x_ls);
        }
        #pragma unroll
        for (int u = 0; u < kUpdUnroll; ++u) {
            if (t + u < L) {
                const int i = t + u;
                if (kCirc) {
                    *reinterpret_cast<uint4 *>(sp + wr * a.s_ls) = raw[u];
                    wr = wr + 1 >= S ? 0 : wr + 1;
                } else if (!in_regs) {
                    const int r = S - L + i;
                    if (r >= 0) *reinterpret_cast<uint4 *>(sp + r * a.s_ls) = raw[u];
                }
                float cur[C], o[C];
                unpack<T>(raw[u], cur);
                #pragma unroll
                for (int c = 0; c < C; ++c) {
                    float acc = bv[c];
                    #pragma unroll
                    for (int k = 0; k < W - 1; ++k) acc = fmaf(wv[k][c], win[k][c], acc);
                    acc = fmaf(wv[W - 1][c], cur[c], acc);
                    o[c] = kSilu ? silu_f(acc) : acc;
                }
                st_stream(op + i * a.o_ls, pack<T>(o));
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
    if (in_regs) {
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) *reinterpret_cast<uint4 *>(sp + k * a.s_ls) = pack<T>(win[k]);
    }
}

template <typename T, int W, bool kSilu, bool kCirc>
__global__ void __launch_bounds__(128) update_generic_kernel(const UpdArgs a) {
    const int64_t c = (int64_t)(blockIdx.x % a.ncolblk) * 128 + threadIdx.x;
    const int32_t b = blockIdx.x / a.ncolblk;
    if (c >= a.dim) return;
    const T *__restrict__ xp = reinterpret_cast<const T *>(a.x) + b * a.x_bs + c * a.x_cs;
    T *__restrict__ op = reinterpret_cast<T *>(a.out) + b * a.o_bs + c * a.o_cs;
    const int L = a.seqlen, S = a.state_len;
    const int32_t coord = a.indices != nullptr ? a.indices[b] : b;
    if (coord < 0) {
        for (int i = 0; i < L; ++i) op[i * a.o_ls] = Elem<T>::from_f(0.f);
        return;
    }
    T *sp = reinterpret_cast<T *>(a.state) + coord * a.s_bs + c * a.s_cs;
    float wv[W];
    #pragma unroll
    for (int k = 0; k < W; ++k) wv[k] = load_w(a.weight, c * a.w_cs + k * a.w_ws, a.wtype);
    const float bv = a.bias != nullptr ? load_w(a.bias, c, a.wtype) : 0.f;

    float win[W - 1];
    int wr = 0;
    if (kCirc) {
        wr = a.cache_seqlens[b] % S;
        if (wr < 0) wr += S;
        int r = wr - (W - 1);
        if (r < 0) r += S;
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) { win[k] = Elem<T>::to_f(sp[r * a.s_ls]); r = r + 1 >= S ? r + 1 - S : r + 1; }
    } else {
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) win[k] = Elem<T>::to_f(sp[(S - (W - 1) + k) * a.s_ls]);
        for (int i = 0; i < S - L; ++i) sp[i * a.s_ls] = sp[(i + L) * a.s_ls];
    }
    for (int i = 0; i < L; ++i) {
        const T xv = xp[i * a.x_ls];
        if (kCirc) {
            sp[wr * a.s_ls] = xv;
            wr = wr + 1 >= S ? 0 : wr + 1;
        } else if (S - L + i >= 0) {
            sp[(S - L + i) * a.s_ls] = xv;
        }
        const float cur = Elem<T>::to_f(xv);
        float acc = bv;
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) acc = fmaf(wv[k], win[k], acc);
        acc = fmaf(wv[W - 1], cur, acc);
        op[i * a.o_ls] = Elem<T>::from_f(kSilu ? silu_f(acc) : acc);
        #pragma unroll
        for (int k = 0; k < W - 2; ++k) win[k] = win[k + 1];
        win[W - 2] = cur;
    }
}

int launch_update(const cc1d_update_params &p, cudaStream_t stream) {
    if (p.batch == 0 || p.dim == 0 || p.seqlen == 0) return CC1D_OK;
    if (p.batch >= (1ll << 31) || p.seqlen >= (1ll << 31) || p.conv_state_len >= (1ll << 31))
        return CC1D_ERR_TOO_LARGE;
    const int C = vec_elems(p.itype);
    UpdArgs a;
    a.x = p.x; a.out = p.out; a.state = p.conv_state; a.weight = p.weight; a.bias = p.bias;
    a.cache_seqlens = p.cache_seqlens; a.indices = p.conv_state_indices;
    a.x_bs = p.x_batch_stride; a.x_cs = p.x_c_stride; a.x_ls = p.x_l_stride;
    a.o_bs = p.out_batch_stride; a.o_cs = p.out_c_stride; a.o_ls = p.out_l_stride;
    a.s_bs = p.conv_state_batch_stride; a.s_cs = p.conv_state_c_stride; a.s_ls = p.conv_state_l_stride;
    a.w_cs = p.weight_c_stride; a.w_ws = p.weight_width_stride;
    a.dim = p.dim; a.batch = (int32_t)p.batch; a.seqlen = (int32_t)p.seqlen;
    a.state_len = (int32_t)p.conv_state_len; a.wtype = p.wtype;

    // a stride only matters when its extent exceeds 1
    const int64_t x_ls = p.seqlen > 1 ? p.x_l_stride : 0, o_ls = p.seqlen > 1 ? p.out_l_stride : 0;
    const int64_t x_bs = p.batch > 1 ? p.x_batch_stride : 0, o_bs = p.batch > 1 ? p.out_batch_stride : 0;
    const int64_t s_ls = p.conv_state_len > 1 ? p.conv_state_l_stride : 0;
    const bool vec_ok = p.dim % C == 0 && (p.dim == 1 || (p.x_c_stride == 1 && p.out_c_stride == 1 &&
                                                          p.conv_state_c_stride == 1)) &&
                        is_aligned16(p.x) && is_aligned16(p.out) && is_aligned16(p.conv_state) &&
                        x_ls % C == 0 && o_ls % C == 0 && x_bs % C == 0 && o_bs % C == 0 && s_ls % C == 0 &&
                        p.conv_state_batch_stride % C == 0;
    const bool circ = p.cache_seqlens != nullptr;
    if (vec_ok) {
        a.ncols = (uint32_t)(p.dim / C);
        a.ncolblk = (a.ncols + 31) / 32;
        const uint64_t ctas = (uint64_t)a.ncolblk * (uint64_t)((p.batch + kUpdRows - 1) / kUpdRows);
        if (ctas >= (1ull << 31)) return CC1D_ERR_TOO_LARGE;
        CC1D_DISPATCH_ITYPE(p.itype, CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu,
            CC1D_DISPATCH_BOOL(circ, kCirc, {
                update_vec_kernel<T, W, kSilu, kCirc><<<(unsigned)ctas, 32 * kUpdRows, 0, stream>>>(a);
            }););););
    } else {
        a.ncols = 0;
        a.ncolblk = (uint32_t)((p.dim + 127) / 128);
        const uint64_t ctas = (uint64_t)a.ncolblk * (uint64_t)p.batch;
        if (ctas >= (1ull << 31)) return CC1D_ERR_TOO_LARGE;
        CC1D_DISPATCH_ITYPE(p.itype, CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu,
            CC1D_DISPATCH_BOOL(circ, kCirc, {
                update_generic_kernel<T, W, kSilu, kCirc><<<(unsigned)ctas, 128, 0, stream>>>(a);
            }););););
    }
    return check_launch();
}

}  // namespace cc1d
