// Decode-step state update kernels (sm_100a).  Replaces causal_conv1d_update_kernel
// (csrc/causal_conv1d_update.cu:23-114 of the reference).
//
// Vector path (x, out and conv_state all have channel stride 1): a thread owns one 16-byte
// vector of channels of one batch entry; a warp touches 512 contiguous bytes per state row /
// token.  The width-1 window is read once; with state_len == width-1 the new state is the
// window left in registers after the last token, otherwise rows are shifted by row copies.
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

// element c of a 16-byte vector as fp32
template <typename T> __device__ __forceinline__ float elem_f(const uint4 &v, int c);
template <> __device__ __forceinline__ float elem_f<float>(const uint4 &v, int c) {
    return __uint_as_float(c == 0 ? v.x : c == 1 ? v.y : c == 2 ? v.z : v.w);
}
template <> __device__ __forceinline__ float elem_f<__nv_bfloat16>(const uint4 &v, int c) {
    const uint32_t w = (c >> 1) == 0 ? v.x : (c >> 1) == 1 ? v.y : (c >> 1) == 2 ? v.z : v.w;
    return __uint_as_float((c & 1) ? (w & 0xffff0000u) : (w << 16));
}
template <> __device__ __forceinline__ float elem_f<__half>(const uint4 &v, int c) {
    const uint32_t w = (c >> 1) == 0 ? v.x : (c >> 1) == 1 ? v.y : (c >> 1) == 2 ? v.z : v.w;
    const unsigned short h = (unsigned short)((c & 1) ? (w >> 16) : (w & 0xffffu));
    return __half2float(*reinterpret_cast<const __half *>(&h));
}

// One thread: one 16-byte vector of channels of one batch entry.  The kernel is kept small
// and straight (a decode step is latency-bound: instruction fetch, one index -> state-row
// dependent load chain, no barrier): every load that does not depend on the state row index
// (taps, first token, cache_seqlens) is issued before the index arrives; later tokens are
// prefetched one ahead in a rolled loop.
template <typename T, int W, bool kSilu, bool kCirc, int kTok>
__global__ void __launch_bounds__(128, kTok == 1 ? 4 : 5) update_vec_kernel(const UpdArgs a) {
    pdl_wait();
    constexpr int C = Elem<T>::kVec;
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
    // flat thread index over (batch entry, channel vector), channel vectors fastest
    const uint64_t gid = (uint64_t)blockIdx.x * 128 + threadIdx.x;
    const int32_t b = (int32_t)(gid / a.ncols);
    const uint32_t col = (uint32_t)(gid - (uint64_t)b * a.ncols);
    if (b >= a.batch) return;
    const int L = a.seqlen, S = a.state_len;

    const int32_t coord = a.indices != nullptr ? __ldg(a.indices + b) : b;
    const int32_t cs = kCirc ? __ldg(a.cache_seqlens + b) : 0;
    const T *__restrict__ xp = reinterpret_cast<const T *>(a.x) + (int64_t)b * a.x_bs + (int64_t)col * C;
    T *__restrict__ op = reinterpret_cast<T *>(a.out) + (int64_t)b * a.o_bs + (int64_t)col * C;
    uint4 raw = ld_stream(xp);   // token 0
    if (coord < 0) {             // padded entry: zero output, state untouched
        for (int i = 0; i < L; ++i) st_stream(op + i * a.o_ls, make_uint4(0, 0, 0, 0));
        return;
    }
    T *sp = reinterpret_cast<T *>(a.state) + coord * a.s_bs + (int64_t)col * C;

    // window rows: the width-1 entries that precede x
    int wr = 0;   // circular: next row to write
    uint4 winraw[W - 1];
    if (kCirc) {
        wr = cs % S;
        if (wr < 0) wr += S;
        int r = wr - (W - 1);
        if (r < 0) r += S;   // state_len >= width-1
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) { winraw[k] = ld_cached(sp + r * a.s_ls); r = r + 1 >= S ? r + 1 - S : r + 1; }
    } else {
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) winraw[k] = ld_cached(sp + (S - (W - 1) + k) * a.s_ls);
    }
    float wv[W][C], bv[C];
    load_taps<W, C>(wv, bv, a.weight, a.w_cs, a.w_ws, a.bias, a.wtype, (int64_t)col * C, kTanh ? 0.5f : 1.f);

    // linear mode with spare rows: shift the surviving rows down by L (ascending, in place;
    // the window rows are already in registers).  With state_len == width-1 the new state is
    // simply the window left after the last token.
    const bool in_regs = !kCirc && S == W - 1;
    if (!kCirc && !in_regs) {
        #pragma unroll 2
        for (int i = 0; i < S - L; ++i) {
            const uint4 v = ld_cached(sp + (i + L) * a.s_ls);
            *reinterpret_cast<uint4 *>(sp + i * a.s_ls) = v;
        }
    }
    if constexpr (kTok > 1) {
        // tokens in chunks of kTok: all loads of a chunk are requested together (one round trip to
        // memory per chunk instead of one per token); token 0 is already here.  kTok == 1 is the
        // single-token decode step, which wants the smaller register footprint.
        #pragma unroll 1
        for (int i0 = 0; i0 < L; i0 += kTok) {
            uint4 tok[kTok];
            #pragma unroll
            for (int j = 0; j < kTok; ++j) {
                tok[j] = raw;
                if ((j > 0 || i0 > 0) && i0 + j < L) tok[j] = ld_stream(xp + (i0 + j) * a.x_ls);
            }
            #pragma unroll
            for (int j = 0; j < kTok; ++j) {
                const int i = i0 + j;
                if (i < L) {
                    const uint4 cur_raw = tok[j];
                    if (kCirc) {
                        *reinterpret_cast<uint4 *>(sp + wr * a.s_ls) = cur_raw;
                        wr = wr + 1 >= S ? 0 : wr + 1;
                    } else if (!in_regs) {
                        const int r = S - L + i;
                        if (r >= 0) *reinterpret_cast<uint4 *>(sp + r * a.s_ls) = cur_raw;
                    }
                    // the window stays in raw vectors; elements are converted where they are used
                    float o[C];
                    #pragma unroll
                    for (int c = 0; c < C; ++c) {
                        float acc = bv[c];
                        #pragma unroll
                        for (int k = 0; k < W - 1; ++k) acc = fmaf(wv[k][c], elem_f<T>(winraw[k], c), acc);
                        acc = fmaf(wv[W - 1][c], elem_f<T>(cur_raw, c), acc);
                        o[c] = !kSilu ? acc : (kTanh ? silu_half_arg(acc) : silu_f(acc));
                    }
                    st_stream(op + i * a.o_ls, pack<T>(o));
                    #pragma unroll
                    for (int k = 0; k < W - 2; ++k) winraw[k] = winraw[k + 1];
                    winraw[W - 2] = cur_raw;   // bit-exact copy for the state write-back
                }
            }
        }
    } else {
        // the single-token decode step (seqlen == 1): straight code, window elements converted where
        // they are used, so that the thread holds the window only as raw vectors
        if (kCirc) *reinterpret_cast<uint4 *>(sp + wr * a.s_ls) = raw;
        else if (!in_regs) *reinterpret_cast<uint4 *>(sp + (S - 1) * a.s_ls) = raw;
        float o[C];
        #pragma unroll
        for (int c = 0; c < C; ++c) {
            float acc = bv[c];
            #pragma unroll
            for (int k = 0; k < W - 1; ++k) acc = fmaf(wv[k][c], elem_f<T>(winraw[k], c), acc);
            acc = fmaf(wv[W - 1][c], elem_f<T>(raw, c), acc);
            o[c] = !kSilu ? acc : (kTanh ? silu_half_arg(acc) : silu_f(acc));
        }
        st_stream(op, pack<T>(o));
        #pragma unroll
        for (int k = 0; k < W - 2; ++k) winraw[k] = winraw[k + 1];
        winraw[W - 2] = raw;   // bit-exact copies for the state write-back
    }
    if (in_regs) {
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) *reinterpret_cast<uint4 *>(sp + k * a.s_ls) = winraw[k];
    }
}

// ---- channel-first state, single-token decode ------------------------------------------
// conv_state contiguous as (entries, dim, S): the S state elements of a channel are adjacent,
// so the C channels of a thread own C*S contiguous elements = S 16-byte vectors.  They are
// shifted as raw bits in registers (bit-exact by construction) and written back whole.
// Element (c, s) of the thread's block sits at flat index c*S + s.
template <typename T> struct Bits;   // raw element <-> fp32, element extraction from 32-bit registers
template <> struct Bits<float> {
    static __device__ __forceinline__ uint32_t get(const uint32_t *r, int i) { return r[i]; }
    static __device__ __forceinline__ void put(uint32_t *r, int i, uint32_t v) { r[i] = v; }
    static __device__ __forceinline__ float to_f(uint32_t v) { return __uint_as_float(v); }
};
template <> struct Bits<__nv_bfloat16> {
    static __device__ __forceinline__ uint32_t get(const uint32_t *r, int i) { return (i & 1) ? r[i >> 1] >> 16 : r[i >> 1] & 0xffffu; }
    static __device__ __forceinline__ void put(uint32_t *r, int i, uint32_t v) { r[i >> 1] |= (i & 1) ? v << 16 : v; }
    static __device__ __forceinline__ float to_f(uint32_t v) { return __uint_as_float(v << 16); }
};
template <> struct Bits<__half> {
    static __device__ __forceinline__ uint32_t get(const uint32_t *r, int i) { return (i & 1) ? r[i >> 1] >> 16 : r[i >> 1] & 0xffffu; }
    static __device__ __forceinline__ void put(uint32_t *r, int i, uint32_t v) { r[i >> 1] |= (i & 1) ? v << 16 : v; }
    static __device__ __forceinline__ float to_f(uint32_t v) {
        const unsigned short h = (unsigned short)v;
        return __half2float(*reinterpret_cast<const __half *>(&h));
    }
};

template <typename T, int W, bool kSilu, int S>
__global__ void __launch_bounds__(128, 4) update_cfstate_kernel(const UpdArgs a) {
    pdl_wait();
    constexpr int C = Elem<T>::kVec;
    constexpr int kRegs = S * 4;   // C * S elements in 32-bit registers
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
    const uint64_t gid = (uint64_t)blockIdx.x * 128 + threadIdx.x;
    const int32_t b = (int32_t)(gid / a.ncols);
    const uint32_t col = (uint32_t)(gid - (uint64_t)b * a.ncols);
    if (b >= a.batch) return;

    const int32_t coord = a.indices != nullptr ? __ldg(a.indices + b) : b;
    const T *__restrict__ xp = reinterpret_cast<const T *>(a.x) + (int64_t)b * a.x_bs + (int64_t)col * C;
    T *__restrict__ op = reinterpret_cast<T *>(a.out) + (int64_t)b * a.o_bs + (int64_t)col * C;
    const uint4 xraw = ld_stream(xp);
    if (coord < 0) {   // padded entry: zero output, state untouched
        st_stream(op, make_uint4(0, 0, 0, 0));
        return;
    }
    uint4 *sp = reinterpret_cast<uint4 *>(reinterpret_cast<T *>(a.state) + coord * a.s_bs + (int64_t)col * C * S);
    uint4 sv[S];
    #pragma unroll
    for (int i = 0; i < S; ++i) sv[i] = ld_cached(sp + i);
    float wv[W][C], bv[C];
    load_taps<W, C>(wv, bv, a.weight, a.w_cs, a.w_ws, a.bias, a.wtype, (int64_t)col * C, kTanh ? 0.5f : 1.f);

    uint32_t old[kRegs], nw[kRegs], xr[4] = {xraw.x, xraw.y, xraw.z, xraw.w};
    #pragma unroll
    for (int i = 0; i < S; ++i) { old[4 * i] = sv[i].x; old[4 * i + 1] = sv[i].y; old[4 * i + 2] = sv[i].z; old[4 * i + 3] = sv[i].w; }
    #pragma unroll
    for (int i = 0; i < kRegs; ++i) nw[i] = 0;
    float o[C];
    #pragma unroll
    for (int c = 0; c < C; ++c) {
        const uint32_t xb = Bits<T>::get(xr, c);
        float acc = bv[c];
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) acc = fmaf(wv[k][c], Bits<T>::to_f(Bits<T>::get(old, c * S + S - (W - 1) + k)), acc);
        acc = fmaf(wv[W - 1][c], Bits<T>::to_f(xb), acc);
        o[c] = !kSilu ? acc : (kTanh ? silu_half_arg(acc) : silu_f(acc));
        // new state of the channel: the old one shifted by one token, x appended
        #pragma unroll
        for (int t = 0; t < S - 1; ++t) Bits<T>::put(nw, c * S + t, Bits<T>::get(old, c * S + t + 1));
        Bits<T>::put(nw, c * S + S - 1, xb);
    }
    st_stream(op, pack<T>(o));
    #pragma unroll
    for (int i = 0; i < S; ++i) sp[i] = make_uint4(nw[4 * i], nw[4 * i + 1], nw[4 * i + 2], nw[4 * i + 3]);
}

// ---- channel-first state, several tokens and / or the circular buffer (16-bit types) -------------
// Same ownership as update_cfstate_kernel: a thread holds the C = 8 channels x S state elements of
// its block as raw bits in registers.  x and out are channel-major as well for L > 1 (the L tokens of
// a channel adjacent: (batch, dim, L) contiguous), so the thread's tokens are L 16-byte vectors.
//   linear (S == width-1 or width): per channel seq = [state | tokens]; output i is the dot product of
//     the taps with seq[S-(W-1)+i ..]; the new state is seq[L .. L+S).
//   circular (S == 8, one 16-byte vector per channel): one branch on the write position
//     cache_seqlens % 8 (the same for the whole thread, nearly always for the whole warp), so that the
//     window slots and the slots the tokens go to are compile-time positions in every case: no dynamic
//     register indexing, no rotation.
// A circular step rewrites the whole 16-byte row of every channel: the rows are 16 bytes, DRAM moves
// 32-byte sectors, so nothing narrower than the row could be written anyway.
template <typename T> __device__ __forceinline__ uint32_t bits_from_f(float v);
template <> __device__ __forceinline__ uint32_t bits_from_f<__nv_bfloat16>(float v) {
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    return (uint32_t)*reinterpret_cast<const unsigned short *>(&h);
}
template <> __device__ __forceinline__ uint32_t bits_from_f<__half>(float v) {
    const __half h = __float2half_rn(v);
    return (uint32_t)*reinterpret_cast<const unsigned short *>(&h);
}

// The 8 channels of a thread: `old` holds their S state elements each (flat c * S + s), `xr` their L
// tokens (flat c * L + i); fills the new state `nw` and the outputs `ob` (both zero on entry).
// kWr: the circular buffer's write position (linear mode: unused).
template <typename T, int W, bool kSilu, int S, bool kCirc, int L, int kWr>
__device__ __forceinline__ void cfstate_channels(const uint32_t (&old)[S * 4], const uint32_t (&xr)[L * 4],
                                                 const float (&wv)[W][8], const float (&bv)[8], uint32_t (&nw)[S * 4],
                                                 uint32_t (&ob)[L * 4]) {
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
    #pragma unroll
    for (int c = 0; c < 8; ++c) {
        uint32_t seq[W - 1 + L];          // the window, then the tokens
        #pragma unroll
        for (int i = 0; i < L; ++i) seq[W - 1 + i] = Bits<T>::get(xr, c * L + i);
        if (kCirc) {
            // window: the width-1 slots before the write position; tokens go to slots kWr, kWr + 1, ... (mod S)
            #pragma unroll
            for (int k = 0; k < W - 1; ++k) seq[k] = Bits<T>::get(old, c * S + (kWr - (W - 1) + k + S) % S);
            #pragma unroll
            for (int j = 0; j < S; ++j) {
                const int i = (j - kWr + S) % S;      // token index that lands in slot j, if any
                Bits<T>::put(nw, c * S + j, i < L ? seq[W - 1 + (i < L ? i : 0)] : Bits<T>::get(old, c * S + j));
            }
        } else {
            uint32_t all[S + L];
            #pragma unroll
            for (int j = 0; j < S; ++j) all[j] = Bits<T>::get(old, c * S + j);
            #pragma unroll
            for (int i = 0; i < L; ++i) all[S + i] = seq[W - 1 + i];
            #pragma unroll
            for (int k = 0; k < W - 1; ++k) seq[k] = all[S - (W - 1) + k];
            #pragma unroll
            for (int t = 0; t < S; ++t) Bits<T>::put(nw, c * S + t, all[t + L]);
        }
        #pragma unroll
        for (int i = 0; i < L; ++i) {
            float acc = bv[c];
            #pragma unroll
            for (int k = 0; k < W; ++k) acc = fmaf(wv[k][c], Bits<T>::to_f(seq[i + k]), acc);
            const float o = !kSilu ? acc : (kTanh ? silu_half_arg(acc) : silu_f(acc));
            Bits<T>::put(ob, c * L + i, bits_from_f<T>(o));
        }
    }
}

template <typename T, int W, bool kSilu, int S, bool kCirc, int L>
__global__ void __launch_bounds__(128, 4) update_cfstate_multi_kernel(const UpdArgs a) {
    pdl_wait();
    static_assert(sizeof(T) == 2, "16-bit types");
    static_assert(!kCirc || S == 8, "circular mode: 8 slots");
    constexpr int C = 8;
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
    const uint64_t gid = (uint64_t)blockIdx.x * 128 + threadIdx.x;
    const int32_t b = (int32_t)(gid / a.ncols);
    const uint32_t col = (uint32_t)(gid - (uint64_t)b * a.ncols);
    if (b >= a.batch) return;

    const int32_t coord = a.indices != nullptr ? __ldg(a.indices + b) : b;
    const int32_t cs = kCirc ? __ldg(a.cache_seqlens + b) : 0;
    const uint4 *xp = reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(a.x) + (int64_t)b * a.x_bs + (int64_t)col * C * L);
    uint4 *op = reinterpret_cast<uint4 *>(reinterpret_cast<T *>(a.out) + (int64_t)b * a.o_bs + (int64_t)col * C * L);
    uint4 xv[L];
    #pragma unroll
    for (int i = 0; i < L; ++i) xv[i] = ld_stream(xp + i);
    if (coord < 0) {   // padded entry: zero output, state untouched
        #pragma unroll
        for (int i = 0; i < L; ++i) st_stream(op + i, make_uint4(0, 0, 0, 0));
        return;
    }
    uint4 *sp = reinterpret_cast<uint4 *>(reinterpret_cast<T *>(a.state) + coord * a.s_bs + (int64_t)col * C * S);
    uint4 sv[S];
    #pragma unroll
    for (int i = 0; i < S; ++i) sv[i] = ld_cached(sp + i);
    float wv[W][C], bv[C];
    load_taps<W, C>(wv, bv, a.weight, a.w_cs, a.w_ws, a.bias, a.wtype, (int64_t)col * C, kTanh ? 0.5f : 1.f);

    uint32_t old[S * 4], nw[S * 4], xr[L * 4], ob[L * 4];
    #pragma unroll
    for (int i = 0; i < S; ++i) { old[4 * i] = sv[i].x; old[4 * i + 1] = sv[i].y; old[4 * i + 2] = sv[i].z; old[4 * i + 3] = sv[i].w; }
    #pragma unroll
    for (int i = 0; i < L; ++i) { xr[4 * i] = xv[i].x; xr[4 * i + 1] = xv[i].y; xr[4 * i + 2] = xv[i].z; xr[4 * i + 3] = xv[i].w; }
    #pragma unroll
    for (int i = 0; i < S * 4; ++i) nw[i] = 0;
    #pragma unroll
    for (int i = 0; i < L * 4; ++i) ob[i] = 0;
    if constexpr (kCirc) {
        // The write position is the same for all channels of the thread (and, a few warps apart, of the
        // warp): one branch on it, and every position inside a case is a compile-time constant.
        int wr = cs % S;
        if (wr < 0) wr += S;
        switch (wr) {
            case 0: cfstate_channels<T, W, kSilu, S, true, L, 0>(old, xr, wv, bv, nw, ob); break;
            case 1: cfstate_channels<T, W, kSilu, S, true, L, 1>(old, xr, wv, bv, nw, ob); break;
            case 2: cfstate_channels<T, W, kSilu, S, true, L, 2>(old, xr, wv, bv, nw, ob); break;
            case 3: cfstate_channels<T, W, kSilu, S, true, L, 3>(old, xr, wv, bv, nw, ob); break;
            case 4: cfstate_channels<T, W, kSilu, S, true, L, 4>(old, xr, wv, bv, nw, ob); break;
            case 5: cfstate_channels<T, W, kSilu, S, true, L, 5>(old, xr, wv, bv, nw, ob); break;
            case 6: cfstate_channels<T, W, kSilu, S, true, L, 6>(old, xr, wv, bv, nw, ob); break;
            default: cfstate_channels<T, W, kSilu, S, true, L, 7>(old, xr, wv, bv, nw, ob); break;
        }
    } else {
        cfstate_channels<T, W, kSilu, S, false, L, 0>(old, xr, wv, bv, nw, ob);
    }
    #pragma unroll
    for (int i = 0; i < L; ++i) st_stream(op + i, make_uint4(ob[4 * i], ob[4 * i + 1], ob[4 * i + 2], ob[4 * i + 3]));
    #pragma unroll
    for (int i = 0; i < S; ++i) sp[i] = make_uint4(nw[4 * i], nw[4 * i + 1], nw[4 * i + 2], nw[4 * i + 3]);
}

template <typename T, int W, bool kSilu, bool kCirc>
__global__ void __launch_bounds__(128) update_generic_kernel(const UpdArgs a) {
    pdl_wait();
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
    // contiguous (entries, dim, S) state, one token, S == width-1 or width: whole-block register shift
    const int64_t S = p.conv_state_len;
    const bool cf_state_ok = !circ && p.seqlen == 1 && p.dim % C == 0 && (p.dim == 1 || (p.x_c_stride == 1 && p.out_c_stride == 1)) &&
                             p.conv_state_l_stride == 1 && p.conv_state_c_stride == S && (S == p.width - 1 || S == p.width) &&
                             S >= 2 && is_aligned16(p.x) && is_aligned16(p.out) && is_aligned16(p.conv_state) &&
                             x_bs % C == 0 && o_bs % C == 0 && (p.conv_state_batch_stride * elem_size(p.itype)) % 16 == 0;
    // contiguous (entries, dim, S) state with 16-bit elements, up to 4 tokens (x and out (batch, dim, L)
    // contiguous as well when L > 1): linear with S == width-1 or width, or the circular pool of 8 slots
    const int64_t Lx = p.seqlen;
    const bool x_cm = Lx == 1 ? (p.dim == 1 || (p.x_c_stride == 1 && p.out_c_stride == 1))
                              : (p.x_l_stride == 1 && p.out_l_stride == 1 && (p.dim == 1 || (p.x_c_stride == Lx && p.out_c_stride == Lx)));
    const bool cf_multi_ok = p.itype != CC1D_F32 && Lx >= 1 && Lx <= 4 && p.dim % 8 == 0 && x_cm &&
                             p.conv_state_l_stride == 1 && p.conv_state_c_stride == S &&
                             ((!circ && Lx > 1 && (S == p.width - 1 || S == p.width) && S >= 2) || (circ && S == 8)) &&
                             is_aligned16(p.x) && is_aligned16(p.out) && is_aligned16(p.conv_state) &&
                             x_bs % 8 == 0 && o_bs % 8 == 0 && p.conv_state_batch_stride % 8 == 0;
    if (cf_multi_ok) {
        a.ncols = (uint32_t)(p.dim / 8);
        a.ncolblk = 0;
        const uint64_t ctas = ((uint64_t)a.ncols * (uint64_t)p.batch + 127) / 128;
        if (ctas >= (1ull << 31)) return CC1D_ERR_TOO_LARGE;
#define CC1D_LAUNCH_MULTI(TT, SS, CIRC, LL) \
        launch_k(update_cfstate_multi_kernel<TT, W, kSilu, SS, CIRC, LL>, dim3((unsigned)ctas), dim3(128), 0, stream, a)
#define CC1D_MULTI_BY_L(TT, SS, CIRC) \
        do { if (Lx == 1) { if (CIRC) CC1D_LAUNCH_MULTI(TT, SS, CIRC, (CIRC ? 1 : 2)); } \
             else if (Lx == 2) CC1D_LAUNCH_MULTI(TT, SS, CIRC, 2); \
             else if (Lx == 3) CC1D_LAUNCH_MULTI(TT, SS, CIRC, 3); \
             else CC1D_LAUNCH_MULTI(TT, SS, CIRC, 4); } while (0)
        CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu, {
            if (p.itype == CC1D_BF16) {
                if (circ) CC1D_MULTI_BY_L(__nv_bfloat16, 8, true);
                else if (S == W) CC1D_MULTI_BY_L(__nv_bfloat16, W, false);
                else if (W >= 3) CC1D_MULTI_BY_L(__nv_bfloat16, (W >= 3 ? W - 1 : W), false);
            } else {
                if (circ) CC1D_MULTI_BY_L(__half, 8, true);
                else if (S == W) CC1D_MULTI_BY_L(__half, W, false);
                else if (W >= 3) CC1D_MULTI_BY_L(__half, (W >= 3 ? W - 1 : W), false);
            }
        }););
#undef CC1D_MULTI_BY_L
#undef CC1D_LAUNCH_MULTI
        return check_launch();
    }
    if (cf_state_ok) {
        a.ncols = (uint32_t)(p.dim / C);
        a.ncolblk = 0;
        const uint64_t ctas = ((uint64_t)a.ncols * (uint64_t)p.batch + 127) / 128;
        if (ctas >= (1ull << 31)) return CC1D_ERR_TOO_LARGE;
        const bool s_is_w = S == p.width;
        CC1D_DISPATCH_ITYPE(p.itype, CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu,
            CC1D_DISPATCH_BOOL(s_is_w, kSW, {
                if constexpr (W - 1 + (kSW ? 1 : 0) >= 2) {
                    launch_k(update_cfstate_kernel<T, W, kSilu, W - 1 + (kSW ? 1 : 0)>, dim3((unsigned)ctas), dim3(128), 0, stream, a);
                }
            }););););
        return check_launch();
    }
    if (vec_ok) {
        a.ncols = (uint32_t)(p.dim / C);
        a.ncolblk = 0;
        const uint64_t ctas = ((uint64_t)a.ncols * (uint64_t)p.batch + 127) / 128;
        if (ctas >= (1ull << 31)) return CC1D_ERR_TOO_LARGE;
        CC1D_DISPATCH_ITYPE(p.itype, CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu,
            CC1D_DISPATCH_BOOL(circ, kCirc, {
                if (p.seqlen == 1) launch_k(update_vec_kernel<T, W, kSilu, kCirc, 1>, dim3((unsigned)ctas), dim3(128), 0, stream, a);
                else launch_k(update_vec_kernel<T, W, kSilu, kCirc, 4>, dim3((unsigned)ctas), dim3(128), 0, stream, a);
            }););););
    } else {
        a.ncols = 0;
        a.ncolblk = (uint32_t)((p.dim + 127) / 128);
        const uint64_t ctas = (uint64_t)a.ncolblk * (uint64_t)p.batch;
        if (ctas >= (1ull << 31)) return CC1D_ERR_TOO_LARGE;
        CC1D_DISPATCH_ITYPE(p.itype, CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu,
            CC1D_DISPATCH_BOOL(circ, kCirc, {
                launch_k(update_generic_kernel<T, W, kSilu, kCirc>, dim3((unsigned)ctas), dim3(128), 0, stream, a);
            }););););
    }
    return check_launch();
}

}  // namespace cc1d
