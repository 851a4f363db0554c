// Backward kernels (sm_100a): dx, dweight, dbias, dinitial_states.
//
// Both layouts recompute the pre-activation from x (SiLU case), form
// g = dout * silu'(y), and produce dx as the transposed convolution of g.  dweight/dbias
// are reduced in a fixed order: per-thread fp32 accumulators -> warp shuffle tree (channel-
// first) or fixed-order shared-memory sum over the CTA's token chunks (channel-last) -> one
// partial row per warp unit / CTA in the caller's workspace -> reduce_partials_kernel sums
// the rows in index order.  No float atomics anywhere, so repeated runs are bitwise equal.
// Channel-first rows of 16-bit elements, a multiple of 16 long, on 32-byte aligned rows take
// bwd_cf_wide_kernel (32 bytes per lane, two of the four halos of a vector pair inside the lane).
//
// Replaces csrc/causal_conv1d_bwd.cu:53-259 (channel-first), :329-589 (channel-last) and
// the deterministic-mode workspaces + ATen sums of csrc/causal_conv1d.cpp:388-462.
#include "cc1d_common.cuh"
#include "cc1d_kernels.h"
#include "cc1d_tma.cuh"

namespace cc1d {

// SM count the channel-last tiling is sized for.  A constant, not a device query: the library is built
// for sm_100a (B200, 148 SMs) only, and cc1d_bwd_workspace_bytes() is host-only arithmetic that must
// give the answer the launcher will use even when no device is current.
constexpr int kTilingSMs = 148;

// ======================================================================================
// final reduction of the partial rows
// ======================================================================================
struct ReduceArgs {
    const float *ws;
    float *dweight;
    float *dbias;
    int64_t dw_cs, dw_ws;
    int64_t dim;
    int64_t n_outer, outer_stride;   // e.g. batch
    int64_t n_inner, inner_stride;   // e.g. units per row
    int64_t chan_stride;
    int accumulate;
    // exchange over peer memory (world == 0: none)
    char *peer_base[CC1D_MAX_PEERS];
    int *peer_status;
    int64_t peer_capacity;
    int world, rank;
    uint32_t spin_limit;
};

// One warp per channel.  Lane l sums partial rows l, l+32, ... in ascending order, then a
// fixed xor tree combines the lanes: the summation order never depends on timing.
template <int W>
__global__ void __launch_bounds__(128) reduce_partials_kernel(const ReduceArgs a) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t c = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (c >= a.dim) return;
    float acc[W + 1];
    #pragma unroll
    for (int k = 0; k <= W; ++k) acc[k] = 0.f;
    const int64_t n = a.n_outer * a.n_inner;
    for (int64_t i = lane; i < n; i += 32) {
        const int64_t o = i / a.n_inner, j = i - o * a.n_inner;
        const float *p = a.ws + o * a.outer_stride + c * a.chan_stride + j * a.inner_stride;
        #pragma unroll
        for (int k = 0; k <= W; ++k) acc[k] += p[k];
    }
    #pragma unroll
    for (int k = 0; k <= W; ++k) {
        #pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc[k] += __shfl_xor_sync(kFullMask, acc[k], off);
    }
    if (lane == 0) {
        #pragma unroll
        for (int k = 0; k < W; ++k) {
            float *d = a.dweight + c * a.dw_cs + k * a.dw_ws;
            *d = a.accumulate ? *d + acc[k] : acc[k];
        }
        if (a.dbias != nullptr) a.dbias[c] = a.accumulate ? a.dbias[c] + acc[W] : acc[W];
    }
}

// The same finishing reduction fused with the exchange between the ranks of a batch-sharded
// backward: lane k of a channel's warp owns output k of that channel (taps 0..W-1, then the
// bias); it stores {value, epoch} as one 8-byte line into slot [epoch & 1][rank] of EVERY rank's
// exchange buffer (plain peer stores), then polls the world's slots in its own buffer until the
// stamp equals the epoch (bounded) and adds the values in rank order.  No flag, no fence, no
// read from peer memory.  The epoch of an element is one more than the newest stamp this rank
// left at that element, so nothing has to count calls and a captured graph can be replayed.
// Buffer: [header 4096 B][uint2 lines[2][world][capacity]].
constexpr size_t kPeerHeaderBytesBwd = 4096;
constexpr uint32_t kPeerSpinLimitBwd = 1u << 21;

__device__ __forceinline__ uint2 *peer_lines8(char *base, uint32_t parity, int from_rank, int world, int64_t capacity) {
    return reinterpret_cast<uint2 *>(base + kPeerHeaderBytesBwd) + ((int64_t)parity * world + from_rank) * capacity;
}
__device__ __forceinline__ uint2 ld_line8(const uint2 *p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_line8(uint2 *p, uint32_t value, uint32_t stamp) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" :: "l"(p), "r"(value), "r"(stamp) : "memory");
}

template <int W>
__global__ void __launch_bounds__(128) reduce_partials_exchange_kernel(const ReduceArgs a) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t c = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (c >= a.dim) return;
    float acc[W + 1];
    #pragma unroll
    for (int k = 0; k <= W; ++k) acc[k] = 0.f;
    const int64_t n = a.n_outer * a.n_inner;
    for (int64_t i = lane; i < n; i += 32) {
        const int64_t o = i / a.n_inner, j = i - o * a.n_inner;
        const float *p = a.ws + o * a.outer_stride + c * a.chan_stride + j * a.inner_stride;
        #pragma unroll
        for (int k = 0; k <= W; ++k) acc[k] += p[k];
    }
    #pragma unroll
    for (int k = 0; k <= W; ++k) {
        #pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc[k] += __shfl_xor_sync(kFullMask, acc[k], off);
    }
    if (lane > W) return;
    float mine = acc[0];
    #pragma unroll
    for (int k = 1; k <= W; ++k) mine = lane == k ? acc[k] : mine;
    const int64_t idx = c * (W + 1) + lane;

    const uint32_t last0 = ld_line8(peer_lines8(a.peer_base[a.rank], 0, a.rank, a.world, a.peer_capacity) + idx).y;
    const uint32_t last1 = ld_line8(peer_lines8(a.peer_base[a.rank], 1, a.rank, a.world, a.peer_capacity) + idx).y;
    const uint32_t epoch = (last0 > last1 ? last0 : last1) + 1;
    const uint32_t parity = epoch & 1u;
    for (int r = 0; r < a.world; ++r)
        st_line8(peer_lines8(a.peer_base[r], parity, a.rank, a.world, a.peer_capacity) + idx, __float_as_uint(mine), epoch);
    float sum = 0.f;
    for (int r = 0; r < a.world; ++r) {
        const uint2 *p = peer_lines8(a.peer_base[a.rank], parity, r, a.world, a.peer_capacity) + idx;
        uint2 line = ld_line8(p);
        for (uint32_t it = 0; line.y != epoch && it < a.spin_limit; ++it) {
            __nanosleep(it < 64 ? 20 : 250);
            line = ld_line8(p);
        }
        if (line.y != epoch) {        // the peer never delivered: report, poison this element, stop waiting
            *a.peer_status = 1;
            sum = __uint_as_float(0x7fc00000u);
            break;
        }
        sum = r == 0 ? __uint_as_float(line.x) : sum + __uint_as_float(line.x);
    }
    if (lane < W) {
        float *d = a.dweight + c * a.dw_cs + lane * a.dw_ws;
        *d = a.accumulate ? *d + sum : sum;
    } else if (a.dbias != nullptr) {
        a.dbias[c] = a.accumulate ? a.dbias[c] + sum : sum;
    }
}

static void set_peers(ReduceArgs &r, const cc1d_peer_group *g) {
    r.world = 0; r.rank = 0; r.peer_status = nullptr; r.peer_capacity = 0; r.spin_limit = kPeerSpinLimitBwd;
    for (int i = 0; i < CC1D_MAX_PEERS; ++i) r.peer_base[i] = nullptr;
    if (g == nullptr) return;
    r.world = g->world; r.rank = g->rank; r.peer_status = g->status; r.peer_capacity = g->capacity;
    if (g->spin_limit != 0) r.spin_limit = g->spin_limit;
    for (int i = 0; i < g->world && i < CC1D_MAX_PEERS; ++i) r.peer_base[i] = reinterpret_cast<char *>(g->peer_base[i]);
}

static int launch_reduce(const ReduceArgs &a, int width, cudaStream_t stream) {
    const unsigned grid = (unsigned)((a.dim + 3) / 4);
    if (a.world > 0) {
        CC1D_DISPATCH_WIDTH(width, { launch_k(reduce_partials_exchange_kernel<W>, dim3(grid), dim3(128), 0, stream, a); });
    } else {
        CC1D_DISPATCH_WIDTH(width, { launch_k(reduce_partials_kernel<W>, dim3(grid), dim3(128), 0, stream, a); });
    }
    return check_launch();
}

// ======================================================================================
// channel-first
// ======================================================================================
struct BwdCfArgs {
    const void *x;
    const void *dout;
    void *dx;
    const void *weight;
    const void *bias;
    float *ws;
    int64_t x_bs, x_cs, d_bs, d_cs, o_bs, o_cs, w_cs, w_ws;
    uint32_t dim, seqlen;
    int wtype;
    uint32_t vpr, gpr, gpu, upr, n_units;   // see FwdCfArgs
};

// g = dout * silu'(y) for one element, times ActGrad<kTanh>::kGScale; `v` is the pre-activation
// computed with the taps scaled by ActGrad<kTanh>::kPre (y, or -y/2 for the tanh form).
template <bool kSilu, bool kTanh>
__device__ __forceinline__ float grad_through_act(float dout, float v) {
    if (!kSilu) return dout;
    return kTanh ? act_grad_neg_half_arg(v, dout) : dout * dsilu_f(v);
}

// Shared by both group bodies: g of the first width-1 elements AFTER the unit, recomputed from
// the unit's last x vector (lane 31's xt) and one extra x/dout vector.  Only lane 31 reads it.
template <typename T, int W, bool kSilu, bool kTanh>
__device__ __forceinline__ void seed_right_halo(const uint4 &xlast, const uint4 &xedge, const uint4 &dedge,
                                                const float (&wy)[W], float by, float (&ge)[W - 1]) {
    constexpr int V = Elem<T>::kVec;
    float xt[V], xn[V], dn[V];
    unpack<T>(xlast, xt);
    unpack<T>(xedge, xn);
    unpack<T>(dedge, dn);
    float xx[2 * (W - 1)];
    #pragma unroll
    for (int k = 0; k < W - 1; ++k) { xx[k] = xt[V - (W - 1) + k]; xx[W - 1 + k] = xn[k]; }
    #pragma unroll
    for (int i = 0; i < W - 1; ++i) {
        float y = by;
        #pragma unroll
        for (int k = 0; k < W; ++k) y = fmaf(wy[k], xx[i + k], y);
        ge[i] = grad_through_act<kSilu, kTanh>(dn[i], y);
    }
}

// One group (kVecs vectors per lane), scalar fp32 arithmetic.  Used for fp32 I/O, where the
// kernel is memory-bound and the smaller register footprint matters more than issue slots.
template <typename T, int W, bool kSilu, bool kFull, int kVecs>
__device__ __forceinline__ void bwd_cf_group_scalar(
    const uint4 (&xraw)[kVecs], const uint4 (&draw)[kVecs], const uint4 &carry, bool seed, const uint4 &xedge,
    const uint4 &dedge, const float (&wv)[W], const float (&wy)[W], float by, float (&ge)[W - 1], float (&dw)[W],
    float &db, T *__restrict__ dxr, uint32_t e0, uint32_t L, int lane) {
    constexpr int V = Elem<T>::kVec;
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
    // pass 1: g, dweight, dbias (elements past the row end have dout == 0, so g == 0)
    float gg[kVecs][V];
    #pragma unroll
    for (int j = 0; j < kVecs; ++j) {
        const uint4 prev = prev_vector_tail<V, W>(xraw[j], j > 0 ? xraw[j - 1] : carry, lane);
        float xx[W - 1 + V];
        {
            float pf[V];
            unpack<T>(prev, pf);
            #pragma unroll
            for (int k = 0; k < W - 1; ++k) xx[k] = pf[V - (W - 1) + k];
        }
        unpack<T>(xraw[j], xx + (W - 1));
        unpack<T>(draw[j], gg[j]);
        #pragma unroll
        for (int i = 0; i < V; ++i) {
            if (kSilu) {
                float y = by;
                #pragma unroll
                for (int k = 0; k < W; ++k) y = fmaf(wy[k], xx[i + k], y);
                gg[j][i] = grad_through_act<kSilu, kTanh>(gg[j][i], y);
            }
            db += gg[j][i];
            #pragma unroll
            for (int k = 0; k < W; ++k) dw[k] = fmaf(xx[i + k], gg[j][i], dw[k]);
        }
    }
    if (seed) seed_right_halo<T, W, kSilu, kTanh>(xraw[kVecs - 1], xedge, dedge, wy, by, ge);   // warp-uniform

    // pass 2: dx[t] = sum_k w[k] * g[t + (W-1-k)]
    const int dst_lane = (lane + 1) & 31;
    #pragma unroll
    for (int j = 0; j < kVecs; ++j) {
        float gx[V + W - 1];
        #pragma unroll
        for (int i = 0; i < V; ++i) gx[i] = gg[j][i];
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) {
            // lane l takes lane l+1's g[j][k]; lane 31 takes lane 0's g[j+1][k]
            const float send = (lane == 0 && j + 1 < kVecs) ? gg[j + 1 < kVecs ? j + 1 : j][k] : gg[j][k];
            float r = __shfl_sync(kFullMask, send, dst_lane);
            if (j == kVecs - 1 && lane == 31) r = ge[k];
            gx[V + k] = r;
        }
        const uint32_t e = e0 + j * 32 * V;
        if (!kFull && e >= L) continue;
        float o[V];
        #pragma unroll
        for (int i = 0; i < V; ++i) {
            float acc = 0.f;
            #pragma unroll
            for (int k = 0; k < W; ++k) acc = fmaf(wv[k], gx[i + (W - 1 - k)], acc);
            o[i] = acc;
        }
        store_row_vec<T, kFull>(dxr, e, L, o);
    }
    // the next (lower) group's right halo is this group's first elements, in lane 0
    #pragma unroll
    for (int k = 0; k < W - 1; ++k) ge[k] = __shfl_sync(kFullMask, gg[0][k], 0);
}

// Same group, arithmetic on fp32 pairs (FFMA2): vectors 2*jp and 2*jp+1 of a lane share a
// pair (.x / .y), so every multiply-add covers two elements per issue slot.  Used for 16-bit
// I/O, where the kernel is issue-bound.  dw2/db2 hold per-component partial sums.
template <typename T, int W, bool kSilu, bool kFull, int kVecs>
__device__ __forceinline__ void bwd_cf_group_pairs(
    const uint4 (&xraw)[kVecs], const uint4 (&draw)[kVecs], const uint4 &carry, bool seed, const uint4 &xedge,
    const uint4 &dedge, const float (&wv)[W], const float (&wy)[W], float by, float (&ge)[W - 1], float2 (&dw2)[W],
    float2 &db2, T *__restrict__ dxr, uint32_t e0, uint32_t L, int lane) {
    constexpr int V = Elem<T>::kVec;
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
    if (seed) seed_right_halo<T, W, kSilu, kTanh>(xraw[kVecs - 1], xedge, dedge, wy, by, ge);   // warp-uniform
    const int dst_lane = (lane + 1) & 31;
    // Vector pairs are walked from the last to the first, g and dx of a pair in one go: dx needs
    // g of the width-1 elements after each vector, which are the first elements of the next
    // lane's vector, or (lane 31) of lane 0's next vector — the other half of the pair, the
    // pair done just before (kept in gfirst), or the group after this one (ge).
    float gfirst[W - 1];
    #pragma unroll
    for (int k = 0; k < W - 1; ++k) gfirst[k] = 0.f;
    #pragma unroll
    for (int jp = kVecs / 2 - 1; jp >= 0; --jp) {
        const int j0 = 2 * jp, j1 = 2 * jp + 1;
        const uint4 prev0 = prev_vector_tail<V, W>(xraw[j0], j0 > 0 ? xraw[j0 - 1] : carry, lane);
        const uint4 prev1 = prev_vector_tail<V, W>(xraw[j1], xraw[j0], lane);
        float2 xx[W - 1 + V], gx[V + W - 1];
        {
            float p0[V], p1[V], a0[V], a1[V], d0[V], d1[V];
            unpack<T>(prev0, p0); unpack<T>(prev1, p1);
            unpack<T>(xraw[j0], a0); unpack<T>(xraw[j1], a1);
            unpack<T>(draw[j0], d0); unpack<T>(draw[j1], d1);
            #pragma unroll
            for (int k = 0; k < W - 1; ++k) xx[k] = make_float2(p0[V - (W - 1) + k], p1[V - (W - 1) + k]);
            #pragma unroll
            for (int i = 0; i < V; ++i) { xx[W - 1 + i] = make_float2(a0[i], a1[i]); gx[i] = make_float2(d0[i], d1[i]); }
        }
        #pragma unroll
        for (int i = 0; i < V; ++i) {
            if (kSilu) {
                float2 y = splat2(by);
                #pragma unroll
                for (int k = 0; k < W; ++k) y = fma2(splat2(wy[k]), xx[i + k], y);
                gx[i] = act_grad_pair<kTanh>(y, gx[i]);
            }
            db2 = add2(db2, gx[i]);
            #pragma unroll
            for (int k = 0; k < W; ++k) dw2[k] = fma2(xx[i + k], gx[i], dw2[k]);
        }
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) {
            // lane l takes lane l+1's first elements; lane 31 takes lane 0's next vector
            const float r0 = __shfl_sync(kFullMask, lane == 0 ? gx[k].y : gx[k].x, dst_lane);
            float r1 = __shfl_sync(kFullMask, (lane == 0 && j1 + 1 < kVecs) ? gfirst[k] : gx[k].y, dst_lane);
            if (j1 == kVecs - 1 && lane == 31) r1 = ge[k];
            gx[V + k] = make_float2(r0, r1);
            gfirst[k] = gx[k].x;
        }
        float o0[V], o1[V];
        #pragma unroll
        for (int i = 0; i < V; ++i) {
            float2 acc = make_float2(0.f, 0.f);
            #pragma unroll
            for (int k = 0; k < W; ++k) acc = fma2(splat2(wv[k]), gx[i + (W - 1 - k)], acc);
            o0[i] = acc.x; o1[i] = acc.y;
        }
        const uint32_t ea = e0 + (2 * jp) * 32 * V, eb = ea + 32 * V;
        if (kFull || ea < L) store_row_vec<T, kFull>(dxr, ea, L, o0);
        if (kFull || eb < L) store_row_vec<T, kFull>(dxr, eb, L, o1);
    }
    // the next (lower) group's right halo is this group's first elements, in lane 0
    #pragma unroll
    for (int k = 0; k < W - 1; ++k) ge[k] = __shfl_sync(kFullMask, gfirst[k], 0);
}

// A warp unit is `gpu` consecutive groups of 32 * kVecs vectors of one row, walked BACK to
// front: dx of a group needs g of the first width-1 elements of the group after it, which
// the previous iteration left in lane 0's registers; only the unit's last group has to
// recompute them from one extra x/dout vector.  dweight/dbias accumulate over the whole
// unit: one partial row per unit.
// kFull: seqlen is a multiple of the vector width and every group has all 32 * kVecs vectors.
#ifndef CC1D_BWD_CF_MINBLK
#define CC1D_BWD_CF_MINBLK 3
#endif
template <typename T, int W, bool kSilu, bool kFull, int kVecs>
__global__ void __launch_bounds__(256, CC1D_BWD_CF_MINBLK) bwd_cf_vec_kernel(const BwdCfArgs a) {
    pdl_wait();
    constexpr int V = Elem<T>::kVec;
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
    constexpr bool kPairs = sizeof(T) == 2;
    constexpr uint32_t kGroupElems = 32 * kVecs * V;
    const int lane = threadIdx.x & 31;
    const uint32_t warps_per_cta = blockDim.x >> 5;
    const uint32_t nwarps = gridDim.x * warps_per_cta;
    const uint32_t L = a.seqlen;

    for (uint32_t unit = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); unit < a.n_units; unit += nwarps) {
        const uint32_t row = unit / a.upr;
        const uint32_t seg = unit - row * a.upr;
        const uint32_t b = row / a.dim;
        const uint32_t c = row - b * a.dim;
        const T *__restrict__ xr = reinterpret_cast<const T *>(a.x) + b * a.x_bs + c * a.x_cs;
        const T *__restrict__ dr = reinterpret_cast<const T *>(a.dout) + b * a.d_bs + c * a.d_cs;
        T *__restrict__ dxr = reinterpret_cast<T *>(a.dx) + b * a.o_bs + c * a.o_cs;
        const uint32_t g0 = seg * a.gpu;
        const uint32_t g1 = g0 + a.gpu < a.gpr ? g0 + a.gpu : a.gpr;

        // taps scaled for dx (g is carried times kGScale) and for the pre-activation recompute
        float wv[W], wy[W];
        constexpr float pre = ActGrad<kTanh>::kPre, post = 1.f / ActGrad<kTanh>::kGScale;
        #pragma unroll
        for (int k = 0; k < W; ++k) {
            const float w = load_w(a.weight, c * a.w_cs + k * a.w_ws, a.wtype);
            wv[k] = post * w;
            wy[k] = pre * w;
        }
        const float by = a.bias != nullptr ? pre * load_w(a.bias, c, a.wtype) : 0.f;

        float dw[W], db = 0.f;
        float2 dw2[W], db2 = make_float2(0.f, 0.f);
        #pragma unroll
        for (int k = 0; k < W; ++k) { dw[k] = 0.f; dw2[k] = make_float2(0.f, 0.f); }
        float ge[W - 1];   // g of the first width-1 elements after the current group
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) ge[k] = 0.f;

        for (uint32_t g = g1; g-- > g0;) {
            const uint32_t e0 = (g * (32 * kVecs) + lane) * V;
            uint4 xraw[kVecs], draw[kVecs];
            #pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                xraw[j] = load_row_vec<T, kFull>(xr, e0 + j * 32 * V, L);
                draw[j] = load_row_vec<T, kFull>(dr, e0 + j * 32 * V, L);
            }
            // x vector before lane 0's first one (held by lane 31 for the shuffle), and for the
            // unit's last group the first vector after it (x and dout) to seed `ge`
            uint4 carry = make_uint4(0, 0, 0, 0), xedge = make_uint4(0, 0, 0, 0), dedge = make_uint4(0, 0, 0, 0);
            if (lane == 31 && g > 0) carry = ld_cached(xr + (e0 - 32 * V));
            const bool seed = g == g1 - 1 && g1 < a.gpr;
            if (seed) {
                const uint32_t en = g1 * kGroupElems;   // first element after the unit
                if (kSilu) xedge = load_row_vec<T, false>(xr, en, L);
                dedge = load_row_vec<T, false>(dr, en, L);
            }
            if constexpr (kPairs) {
                bwd_cf_group_pairs<T, W, kSilu, kFull, kVecs>(xraw, draw, carry, seed, xedge, dedge, wv, wy, by, ge, dw2, db2,
                                                              dxr, e0, L, lane);
            } else {
                bwd_cf_group_scalar<T, W, kSilu, kFull, kVecs>(xraw, draw, carry, seed, xedge, dedge, wv, wy, by, ge, dw, db,
                                                               dxr, e0, L, lane);
            }
        }

        // fold the pair components (16-bit path), then the warp tree (fixed order): one partial
        // row per unit
        if constexpr (kPairs) {
            db = db2.x + db2.y;
            #pragma unroll
            for (int k = 0; k < W; ++k) dw[k] = dw2[k].x + dw2[k].y;
        }
        db *= post;                      // the sums were taken over kGScale * g
        #pragma unroll
        for (int k = 0; k < W; ++k) dw[k] *= post;
        #pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            #pragma unroll
            for (int k = 0; k < W; ++k) dw[k] += __shfl_xor_sync(kFullMask, dw[k], off);
            db += __shfl_xor_sync(kFullMask, db, off);
        }
        if (lane == 0) {
            float *p = a.ws + (uint64_t)unit * (W + 1);
            #pragma unroll
            for (int k = 0; k < W; ++k) p[k] = dw[k];
            p[W] = db;
        }
    }
}

// ---- 16-bit I/O, rows of a multiple of 16 elements, 32-byte aligned: 32 bytes per lane --------
// A lane owns SLOTS of 16 consecutive elements (two 16-byte vectors A, B moved by one 256-bit
// load / store); a warp instruction covers 1 KB of the row.  The fp32 pairs hold (A[i], B[i]),
// so of the four halos a pair of vectors has, two stay inside the lane: B's left x halo is
// A's tail and A's right g halo is B's head.  Only A's left halo (previous lane's B tail, 2
// shuffles) and B's right halo (next lane's A head, width-1 shuffles) cross lanes.  Slots are
// walked back to front; lane 0 keeps g of its first elements for lane 31 of the slot before.
__device__ __forceinline__ void ld_stream32(uint4 &a, uint4 &b, const void *p) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p));
}
__device__ __forceinline__ void st_stream32(void *p, const uint4 &a, const uint4 &b) {
    asm volatile("st.global.cs.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :: "l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w) : "memory");
}

#ifndef CC1D_BWD_WIDE
#define CC1D_BWD_WIDE 1            // 0: never take the 32-bytes-per-lane kernel
#endif
#ifndef CC1D_BWD_WIDE_THREADS
#define CC1D_BWD_WIDE_THREADS 128    // with 5 CTAs per SM: 96 registers, 20 warps per SM
#endif
#ifndef CC1D_BWD_WIDE_MINBLK
#define CC1D_BWD_WIDE_MINBLK 5
#endif
#ifndef CC1D_BWD_WIDE_PERSISTENT
#define CC1D_BWD_WIDE_PERSISTENT 0   // 1: grid = resident CTAs, grid-stride loop over the units; 0: one unit per warp
#endif
#ifndef CC1D_BWD_WIDE_STEP
#define CC1D_BWD_WIDE_STEP 2         // slots loaded, then computed, per step (1 or kCfVecs / 2)
#endif
#ifndef CC1D_BWD_WIDE_PREFETCH
#define CC1D_BWD_WIDE_PREFETCH 0   // 1: the next group's vectors are requested before the current group is computed
#endif
#ifndef CC1D_BWD_WIDE_L2PF
#define CC1D_BWD_WIDE_L2PF 1       // steps asked into L2 ahead of the step being loaded (0: none)
#endif
constexpr int kWideSlots = kCfVecs / 2;       // same group size (and partial rows) as the 16-byte kernel
constexpr uint32_t kWideSlotElems = 32 * 16;

template <int kSlots> struct WideGroup {
    uint4 xa[kSlots], xb[kSlots], da[kSlots], db[kSlots];
    uint32_t cz, cw;          // lane 31: the 4 elements of x before the group (zeros at the row start)
};

// kWhole: every slot of the row is complete; otherwise seqlen is only a multiple of 16, a lane's 16
// elements are either all inside the row or all past its end (then they read as zeros: g = 0 there).
template <typename T, int kSlots, bool kWhole>
__device__ __forceinline__ void wide_load(WideGroup<kSlots> &r, const T *__restrict__ xr, const T *__restrict__ dr,
                                          uint32_t g, int lane, uint32_t L) {
    const uint32_t gs = g * (kSlots * kWideSlotElems);
    #pragma unroll
    for (int j = 0; j < kSlots; ++j) {
        const uint32_t e = gs + j * kWideSlotElems + lane * 16;
        if (kWhole || e < L) {
            ld_stream32(r.xa[j], r.xb[j], xr + e);
            ld_stream32(r.da[j], r.db[j], dr + e);
        } else {
            r.xa[j] = r.xb[j] = r.da[j] = r.db[j] = make_uint4(0, 0, 0, 0);
        }
    }
    r.cz = 0; r.cw = 0;
    if (lane == 31 && g > 0) {
        const uint2 t = *reinterpret_cast<const uint2 *>(xr + gs - 4);
        r.cz = t.x; r.cw = t.y;
    }
}

template <typename T, int W, bool kSilu, int kSlots, bool kWhole>
__device__ __forceinline__ void wide_group(const WideGroup<kSlots> &r, const float (&wv)[W], const float (&wy)[W], float by,
                                           float (&gfirst)[W - 1], float2 (&dw2)[W], float2 &db2, T *__restrict__ dxr,
                                           uint32_t g, int lane, uint32_t L) {
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
    const int src_prev = (lane + 31) & 31, src_next = (lane + 1) & 31;
    const uint32_t gs = g * (kSlots * kWideSlotElems);
    #pragma unroll
    for (int j = kSlots - 1; j >= 0; --j) {
        // left x halo of A: the previous lane's B tail; lane 0 gets what lane 31 holds of the slot before
        const uint32_t oz = j > 0 ? r.xb[j > 0 ? j - 1 : 0].z : r.cz, ow = j > 0 ? r.xb[j > 0 ? j - 1 : 0].w : r.cw;
        uint32_t pz = 0;
        if (W >= 4) pz = __shfl_sync(kFullMask, lane == 31 ? oz : r.xb[j].z, src_prev);
        const uint32_t pw = __shfl_sync(kFullMask, lane == 31 ? ow : r.xb[j].w, src_prev);
        float2 xx[W - 1 + 8], gx[8 + W - 1];
        {
            const float2 pa = unpack_pair<T>(pz), pb = unpack_pair<T>(pw);
            const float p[4] = {pa.x, pa.y, pb.x, pb.y};   // elements 4..7 of the vector before A
            float af[8], bf[8], df[8], ef[8];
            unpack<T>(r.xa[j], af); unpack<T>(r.xb[j], bf); unpack<T>(r.da[j], df); unpack<T>(r.db[j], ef);
            #pragma unroll
            for (int k = 0; k < W - 1; ++k) xx[k] = make_float2(p[4 - (W - 1) + k], af[8 - (W - 1) + k]);
            #pragma unroll
            for (int i = 0; i < 8; ++i) { xx[W - 1 + i] = make_float2(af[i], bf[i]); gx[i] = make_float2(df[i], ef[i]); }
        }
        #pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (kSilu) {
                float2 y = splat2(by);
                #pragma unroll
                for (int k = 0; k < W; ++k) y = fma2(splat2(wy[k]), xx[i + k], y);
                gx[i] = act_grad_pair<kTanh>(y, gx[i]);
            }
            db2 = add2(db2, gx[i]);
            #pragma unroll
            for (int k = 0; k < W; ++k) dw2[k] = fma2(xx[i + k], gx[i], dw2[k]);
        }
        // right g halo: A's is B's head; B's is the next lane's A head, lane 31 takes lane 0's from
        // the slot done just before (gfirst), which then moves on to this slot's
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) {
            const float nb = __shfl_sync(kFullMask, lane == 0 ? gfirst[k] : gx[k].x, src_next);
            gfirst[k] = gx[k].x;
            gx[8 + k] = make_float2(gx[k].y, nb);
        }
        float o0[8], o1[8];
        #pragma unroll
        for (int i = 0; i < 8; ++i) {
            float2 acc = make_float2(0.f, 0.f);
            #pragma unroll
            for (int k = 0; k < W; ++k) acc = fma2(splat2(wv[k]), gx[i + (W - 1 - k)], acc);
            o0[i] = acc.x; o1[i] = acc.y;
        }
        const uint32_t e = gs + j * kWideSlotElems + lane * 16;
        if (kWhole || e < L) st_stream32(dxr + e, pack<T>(o0), pack<T>(o1));
    }
}

template <typename T, int W, bool kSilu, int kSlots, bool kPrefetch, bool kWhole>
__global__ void __launch_bounds__(CC1D_BWD_WIDE_THREADS, CC1D_BWD_WIDE_MINBLK) bwd_cf_wide_kernel(const BwdCfArgs a) {
    pdl_wait();
    static_assert(sizeof(T) == 2, "16-bit I/O only");
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
    constexpr uint32_t kGroupElems = kSlots * kWideSlotElems;
    const int lane = threadIdx.x & 31;
    const uint32_t warps_per_cta = blockDim.x >> 5;
    const uint32_t nwarps = gridDim.x * warps_per_cta;

    for (uint32_t unit = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); unit < a.n_units; unit += nwarps) {
        const uint32_t row = unit / a.upr;
        const uint32_t seg = unit - row * a.upr;
        const uint32_t b = row / a.dim;
        const uint32_t c = row - b * a.dim;
        const T *__restrict__ xr = reinterpret_cast<const T *>(a.x) + b * a.x_bs + c * a.x_cs;
        const T *__restrict__ dr = reinterpret_cast<const T *>(a.dout) + b * a.d_bs + c * a.d_cs;
        T *__restrict__ dxr = reinterpret_cast<T *>(a.dx) + b * a.o_bs + c * a.o_cs;
        const uint32_t g0 = seg * a.gpu;
        const uint32_t g1 = g0 + a.gpu < a.gpr ? g0 + a.gpu : a.gpr;

        // first loads requested before the taps are: kPrefetch walks the unit slot by slot with the
        // next slot's vectors already in flight, otherwise a whole group is loaded, then computed
        constexpr int kStep = kPrefetch ? 1 : (CC1D_BWD_WIDE_STEP < kSlots ? CC1D_BWD_WIDE_STEP : kSlots);   // slots per load/compute step
        const uint32_t s0 = g0 * (kSlots / kStep), s1 = g1 * (kSlots / kStep);
        WideGroup<kStep> cur;
        wide_load<T, kStep, kWhole>(cur, xr, dr, s1 - 1, lane, a.seqlen);
        // A warp cannot hold the next step's vectors in registers while it computes this one, so its loads
        // come after the arithmetic and would wait on DRAM; instead the step after the one being loaded is
        // asked into L2, where those loads then find it: one 128-byte line per lane, lanes 0-15 the 2 KB of
        // x, lanes 16-31 the 2 KB of dout.  Holds no register and no shared memory.
        auto prefetch_step = [&](uint32_t s) {
            if (CC1D_BWD_WIDE_L2PF > 0 && !kPrefetch) {
                static_assert(kPrefetch || kStep * kWideSlotElems * sizeof(T) == 16 * 128, "16 lines per tensor and step");
                const uint32_t e = s * (kStep * kWideSlotElems) + (lane & 15) * 64;
                const T *p = (lane < 16 ? xr : dr) + e;
                if (kWhole || e < a.seqlen) asm volatile("prefetch.global.L2 [%0];" :: "l"(p));
            }
        };
        #pragma unroll
        for (uint32_t d = 1; d <= CC1D_BWD_WIDE_L2PF; ++d) {
            if (s1 - 1 >= s0 + d) prefetch_step(s1 - 1 - d);
        }

        float wv[W], wy[W];
        constexpr float pre = ActGrad<kTanh>::kPre, post = 1.f / ActGrad<kTanh>::kGScale;
        #pragma unroll
        for (int k = 0; k < W; ++k) {
            const float w = load_w(a.weight, c * a.w_cs + k * a.w_ws, a.wtype);
            wv[k] = post * w;
            wy[k] = pre * w;
        }
        const float by = a.bias != nullptr ? pre * load_w(a.bias, c, a.wtype) : 0.f;

        float2 dw2[W], db2 = make_float2(0.f, 0.f);
        #pragma unroll
        for (int k = 0; k < W; ++k) dw2[k] = make_float2(0.f, 0.f);
        // g of the first width-1 elements after the unit (zero past the row end), same in all lanes
        float gfirst[W - 1];
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) gfirst[k] = 0.f;
        if (g1 < a.gpr) {   // warp-uniform
            const uint32_t en = g1 * kGroupElems;
            uint4 xlast = make_uint4(0, 0, 0, 0), xedge = make_uint4(0, 0, 0, 0);
            if (kSilu) { xlast = ld_cached(xr + en - 8); xedge = ld_cached(xr + en); }
            const uint4 dedge = ld_cached(dr + en);
            seed_right_halo<T, W, kSilu, kTanh>(xlast, xedge, dedge, wy, by, gfirst);
        }

        if constexpr (kPrefetch) {
            WideGroup<kStep> nxt;
            uint32_t s = s1 - 1;
            while (true) {
                if (s > s0) wide_load<T, kStep, kWhole>(nxt, xr, dr, s - 1, lane, a.seqlen);
                wide_group<T, W, kSilu, kStep, kWhole>(cur, wv, wy, by, gfirst, dw2, db2, dxr, s, lane, a.seqlen);
                if (s == s0) break;
                --s;
                if (s > s0) wide_load<T, kStep, kWhole>(cur, xr, dr, s - 1, lane, a.seqlen);
                wide_group<T, W, kSilu, kStep, kWhole>(nxt, wv, wy, by, gfirst, dw2, db2, dxr, s, lane, a.seqlen);
                if (s == s0) break;
                --s;
            }
        } else {
            for (uint32_t s = s1 - 1;; --s) {
                wide_group<T, W, kSilu, kStep, kWhole>(cur, wv, wy, by, gfirst, dw2, db2, dxr, s, lane, a.seqlen);
                if (s == s0) break;
                wide_load<T, kStep, kWhole>(cur, xr, dr, s - 1, lane, a.seqlen);
                if (s - 1 >= s0 + CC1D_BWD_WIDE_L2PF) prefetch_step(s - 1 - CC1D_BWD_WIDE_L2PF);
            }
        }

        // fold the pair components, then the warp tree (fixed order): one partial row per unit
        float dw[W], db = (db2.x + db2.y) * post;      // the sums were taken over kGScale * g
        #pragma unroll
        for (int k = 0; k < W; ++k) dw[k] = (dw2[k].x + dw2[k].y) * post;
        #pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            #pragma unroll
            for (int k = 0; k < W; ++k) dw[k] += __shfl_xor_sync(kFullMask, dw[k], off);
            db += __shfl_xor_sync(kFullMask, db, off);
        }
        if (lane == 0) {
            float *p = a.ws + (uint64_t)unit * (W + 1);
            #pragma unroll
            for (int k = 0; k < W; ++k) p[k] = dw[k];
            p[W] = db;
        }
    }
}

// Any alignment: one (row, 256-element tile) per CTA, a thread per element; block tree in
// shared memory.  Partial row per tile.
template <typename T, int W, bool kSilu>
__global__ void __launch_bounds__(256) bwd_cf_scalar_kernel(const BwdCfArgs a) {
    pdl_wait();
    __shared__ float red[8][W + 1];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (uint32_t tile = blockIdx.x; tile < a.n_units; tile += gridDim.x) {
        const uint32_t row = tile / a.vpr;
        const int64_t t = (int64_t)(tile - row * a.vpr) * 256 + threadIdx.x;
        const uint32_t b = row / a.dim;
        const uint32_t c = row - b * a.dim;
        const T *__restrict__ xr = reinterpret_cast<const T *>(a.x) + b * a.x_bs + c * a.x_cs;
        const T *__restrict__ dr = reinterpret_cast<const T *>(a.dout) + b * a.d_bs + c * a.d_cs;
        T *__restrict__ dxr = reinterpret_cast<T *>(a.dx) + b * a.o_bs + c * a.o_cs;
        float wv[W];
        #pragma unroll
        for (int k = 0; k < W; ++k) wv[k] = load_w(a.weight, c * a.w_cs + k * a.w_ws, a.wtype);
        const float bv = a.bias != nullptr ? load_w(a.bias, c, a.wtype) : 0.f;
        const int64_t L = a.seqlen;
        // g at t .. t+W-1 (each needs x at s-(W-1) .. s)
        float xs[2 * W - 1];
        #pragma unroll
        for (int i = 0; i < 2 * W - 1; ++i) {
            const int64_t p = t - (W - 1) + i;
            xs[i] = (p >= 0 && p < L) ? Elem<T>::to_f(xr[p]) : 0.f;
        }
        float gs[W];
        #pragma unroll
        for (int m = 0; m < W; ++m) {
            const int64_t s = t + m;
            float gv = s < L ? Elem<T>::to_f(dr[s]) : 0.f;
            if (kSilu) {
                float y = bv;
                #pragma unroll
                for (int k = 0; k < W; ++k) y = fmaf(wv[k], xs[m + k], y);
                gv *= dsilu_f(y);
            }
            gs[m] = gv;
        }
        float dw[W], db = 0.f;
        #pragma unroll
        for (int k = 0; k < W; ++k) dw[k] = 0.f;
        if (t < L) {
            float acc = 0.f;
            #pragma unroll
            for (int k = 0; k < W; ++k) acc = fmaf(wv[k], gs[W - 1 - k], acc);
            dxr[t] = Elem<T>::from_f(acc);
            db = gs[0];
            #pragma unroll
            for (int k = 0; k < W; ++k) dw[k] = xs[k] * gs[0];
        }
        #pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            #pragma unroll
            for (int k = 0; k < W; ++k) dw[k] += __shfl_xor_sync(kFullMask, dw[k], off);
            db += __shfl_xor_sync(kFullMask, db, off);
        }
        __syncthreads();   // previous tile's readers are done with `red`
        if (lane == 0) {
            #pragma unroll
            for (int k = 0; k < W; ++k) red[wid][k] = dw[k];
            red[wid][W] = db;
        }
        __syncthreads();
        if (threadIdx.x <= W) {
            float s = 0.f;
            #pragma unroll
            for (int w8 = 0; w8 < 8; ++w8) s += red[w8][threadIdx.x];
            a.ws[(uint64_t)tile * (W + 1) + threadIdx.x] = s;
        }
    }
}

struct CfPlan {
    bool vec;
    uint64_t vpr, gpr, gpu, upr, n_units;
};

static CfPlan plan_channel_first(const cc1d_bwd_params &p) {
    constexpr int kVecs = kCfVecs;
    const int V = vec_elems(p.itype);
    const int64_t x_bs = p.batch > 1 ? p.x_batch_stride : 0, x_cs = p.dim > 1 ? p.x_c_stride : 0;
    const int64_t d_bs = p.batch > 1 ? p.dout_batch_stride : 0, d_cs = p.dim > 1 ? p.dout_c_stride : 0;
    const int64_t o_bs = p.batch > 1 ? p.dx_batch_stride : 0, o_cs = p.dim > 1 ? p.dx_c_stride : 0;
    CfPlan pl;
    pl.vec = is_aligned16(p.x) && is_aligned16(p.dout) && is_aligned16(p.dx) && x_bs % V == 0 && x_cs % V == 0 &&
             d_bs % V == 0 && d_cs % V == 0 && o_bs % V == 0 && o_cs % V == 0;
    const uint64_t rows = (uint64_t)p.batch * (uint64_t)p.dim;
    if (pl.vec) {
        pl.vpr = ((uint64_t)p.seqlen + V - 1) / V;
        pl.gpr = (pl.vpr + 32 * kVecs - 1) / (32 * kVecs);
        pl.gpu = groups_per_unit(rows, pl.gpr);
        pl.upr = (pl.gpr + pl.gpu - 1) / pl.gpu;
    } else {
        pl.vpr = ((uint64_t)p.seqlen + 255) / 256;
        pl.gpr = pl.gpu = 0;
        pl.upr = pl.vpr;
    }
    pl.n_units = rows * pl.upr;
    return pl;
}

size_t bwd_workspace_bytes_channel_first(const cc1d_bwd_params &p) {
    // Alignment of the data pointers decides vector vs scalar tiling; size for the larger of
    // the two so that the answer does not depend on pointers the caller has not allocated yet.
    const int V = vec_elems(p.itype);
    const uint64_t rows = (uint64_t)p.batch * (uint64_t)p.dim;
    const uint64_t vpr = ((uint64_t)p.seqlen + V - 1) / V;
    const uint64_t gpr = (vpr + kCfGroupVecs - 1) / kCfGroupVecs;
    const uint64_t gpu = groups_per_unit(rows, gpr);
    const uint64_t upr_vec = gpu ? (gpr + gpu - 1) / gpu : 0;
    const uint64_t upr_sc = ((uint64_t)p.seqlen + 255) / 256;
    const uint64_t upr = upr_vec > upr_sc ? upr_vec : upr_sc;
    return (size_t)(rows * upr * (uint64_t)(p.width + 1) * sizeof(float));
}

int launch_bwd_channel_first(const cc1d_bwd_params &p, cudaStream_t stream) {
    const uint64_t rows = (uint64_t)p.batch * (uint64_t)p.dim;
    if (p.seqlen >= (1ll << 31) - 4096 || p.dim >= (1ll << 31)) return CC1D_ERR_TOO_LARGE;
    const CfPlan pl = plan_channel_first(p);
    if (pl.n_units >= (1ull << 31)) return CC1D_ERR_TOO_LARGE;   // unit + grid stride must not wrap 32 bits
    if (pl.n_units * (uint64_t)(p.width + 1) * sizeof(float) > p.workspace_bytes) return CC1D_ERR_WORKSPACE;

    BwdCfArgs a;
    a.x = p.x; a.dout = p.dout; a.dx = p.dx; a.weight = p.weight; a.bias = p.bias;
    a.ws = reinterpret_cast<float *>(p.workspace);
    a.x_bs = p.batch > 1 ? p.x_batch_stride : 0; a.x_cs = p.dim > 1 ? p.x_c_stride : 0;
    a.d_bs = p.batch > 1 ? p.dout_batch_stride : 0; a.d_cs = p.dim > 1 ? p.dout_c_stride : 0;
    a.o_bs = p.batch > 1 ? p.dx_batch_stride : 0; a.o_cs = p.dim > 1 ? p.dx_c_stride : 0;
    a.w_cs = p.weight_c_stride; a.w_ws = p.weight_width_stride;
    a.dim = (uint32_t)p.dim; a.seqlen = (uint32_t)p.seqlen; a.wtype = p.wtype;
    a.vpr = (uint32_t)pl.vpr; a.gpr = (uint32_t)pl.gpr; a.gpu = (uint32_t)pl.gpu; a.upr = (uint32_t)pl.upr;
    a.n_units = (uint32_t)pl.n_units;
    if (rows > 0 && p.seqlen > 0 && p.phase != 2) {
        if (pl.vec) {
            const uint64_t ctas = (pl.n_units + 7) / 8;
            const bool full = p.seqlen % vec_elems(p.itype) == 0 && pl.vpr % kCfGroupVecs == 0;
            // 16-bit rows whose length is a multiple of 16 elements and whose starts are 32-byte aligned: 32
            // bytes per lane (a lane's 16 elements are then never cut by the row end)
            const bool wide = CC1D_BWD_WIDE && kCfVecs % 2 == 0 && p.itype != CC1D_F32 && p.seqlen % 16 == 0 &&
                              ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.dout) |
                                reinterpret_cast<uintptr_t>(p.dx)) & 31u) == 0 &&
                              (a.x_bs | a.x_cs | a.d_bs | a.d_cs | a.o_bs | a.o_cs) % 16 == 0;
            if (wide) {
                const uint64_t wctas = (pl.n_units + CC1D_BWD_WIDE_THREADS / 32 - 1) / (CC1D_BWD_WIDE_THREADS / 32);
                if (p.itype == CC1D_BF16) {
                    using T = __nv_bfloat16;
                    CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu, CC1D_DISPATCH_BOOL(full, kWhole, {
                        auto kernel = bwd_cf_wide_kernel<T, W, kSilu, kWideSlots, CC1D_BWD_WIDE_PREFETCH != 0, kWhole>;
                        launch_k(kernel, dim3(persistent_grid(kernel, CC1D_BWD_WIDE_THREADS, wctas, CC1D_BWD_WIDE_PERSISTENT != 0)),
                                 dim3(CC1D_BWD_WIDE_THREADS), 0, stream, a);
                    });););
                } else {
                    using T = __half;
                    CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu, CC1D_DISPATCH_BOOL(full, kWhole, {
                        auto kernel = bwd_cf_wide_kernel<T, W, kSilu, kWideSlots, CC1D_BWD_WIDE_PREFETCH != 0, kWhole>;
                        launch_k(kernel, dim3(persistent_grid(kernel, CC1D_BWD_WIDE_THREADS, wctas, CC1D_BWD_WIDE_PERSISTENT != 0)),
                                 dim3(CC1D_BWD_WIDE_THREADS), 0, stream, a);
                    });););
                }
            } else
            CC1D_DISPATCH_ITYPE(p.itype, CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu,
                CC1D_DISPATCH_BOOL(full, kFull, {
                    auto kernel = bwd_cf_vec_kernel<T, W, kSilu, kFull, kCfVecs>;
                    const bool persistent = CC1D_CF_BWD_PERSISTENT == 1 || (CC1D_CF_BWD_PERSISTENT == 2 && p.itype != CC1D_F32);
                    launch_k(kernel, dim3(persistent_grid(kernel, 256, ctas, persistent)), dim3(256), 0, stream, a);
                }););););
        } else {
            CC1D_DISPATCH_ITYPE(p.itype, CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu, {
                auto kernel = bwd_cf_scalar_kernel<T, W, kSilu>;
                launch_k(kernel, dim3(persistent_grid(kernel, 256, pl.n_units)), dim3(256), 0, stream, a);
            });););
        }
        if (check_launch() != CC1D_OK) return CC1D_ERR_LAUNCH;
    }
    ReduceArgs r;
    r.ws = a.ws; r.dweight = p.dweight; r.dbias = p.dbias;
    r.dw_cs = p.dweight_c_stride; r.dw_ws = p.dweight_width_stride;
    r.dim = p.dim;
    r.n_outer = (rows > 0 && p.seqlen > 0) ? p.batch : 0;
    r.outer_stride = (int64_t)p.dim * (int64_t)pl.upr * (p.width + 1);
    r.n_inner = (int64_t)pl.upr; r.inner_stride = p.width + 1;
    r.chan_stride = (int64_t)pl.upr * (p.width + 1);
    r.accumulate = p.accumulate;
    set_peers(r, p.peers);
    if (p.dim == 0 || p.phase == 1) return CC1D_OK;
    return launch_reduce(r, p.width, stream);
}

// ======================================================================================
// channel-last
// ======================================================================================
struct BwdClArgs {
    const void *x;
    const void *dout;
    void *dx;
    const void *weight;
    const void *bias;
    const int32_t *seq_idx;
    const void *init;
    const void *dfin;
    void *dinit;
    float *ws;
    int64_t x_bs, x_ls, d_bs, d_ls, o_bs, o_ls, w_cs, w_ws, i_bs, i_ls, df_bs, df_cs, df_ls, di_bs, di_ls;
    int64_t dim, seqlen;
    int wtype;
    int tpt;
    uint32_t ncols, ncolblk, ngroups;
};

#ifndef CC1D_BWD_CL_ROWS
#define CC1D_BWD_CL_ROWS 4
#endif
#ifndef CC1D_BWD_CL_UNROLL
#define CC1D_BWD_CL_UNROLL 4
#endif
#ifndef CC1D_BWD_CL_MINBLK
#define CC1D_BWD_CL_MINBLK 3
#endif
constexpr int kBwdClRows = CC1D_BWD_CL_ROWS;       // token chunks per CTA
constexpr int kBwdClUnroll = CC1D_BWD_CL_UNROLL;   // positions per block (x and dout loads of the next block in flight)
constexpr int kBwdClC = 4;        // channels per thread: 8-byte vectors for 16-bit I/O, 16-byte for fp32

// wy = kPre * w and bv = kPre * bias (pre-activation recompute), wv = w / kGScale (dx): see ActGrad.
template <int W, int C, bool kTanh>
__device__ __forceinline__ void scale_taps_for_backward(float2 (&wv)[W][C / 2], float2 (&wy)[W][C / 2], float2 (&bv)[C / 2]) {
    constexpr float pre = ActGrad<kTanh>::kPre, post = 1.f / ActGrad<kTanh>::kGScale;
    #pragma unroll
    for (int c = 0; c < C / 2; ++c) {
        #pragma unroll
        for (int k = 0; k < W; ++k) {
            wy[k][c] = make_float2(pre * wv[k][c].x, pre * wv[k][c].y);
            wv[k][c] = make_float2(post * wv[k][c].x, post * wv[k][c].y);
        }
        bv[c] = make_float2(pre * bv[c].x, pre * bv[c].y);
    }
}

// the sums were taken over kGScale * g
template <int W, int C, bool kTanh>
__device__ __forceinline__ void unscale_sums(float2 (&dw)[C / 2][W + 1]) {
    if (!kTanh) return;
    constexpr float post = 1.f / ActGrad<kTanh>::kGScale;
    #pragma unroll
    for (int c = 0; c < C / 2; ++c) {
        #pragma unroll
        for (int k = 0; k <= W; ++k) dw[c][k] = make_float2(post * dw[c][k].x, post * dw[c][k].y);
    }
}

// One position `pos` of the backward sliding window (channel-last):
//   g[pos]   = dout[pos] * act'(y[pos])            (y recomputed from the x window)
//   dweight += x window * g[pos], dbias += g[pos]   (only while pos is inside the thread's chunk)
//   dx[q]    = sum_m w[W-1-m] * g[q+m],  q = pos-(W-1)   (stored when q is inside the chunk;
//              for q < 0 the same sum is dinitial_states[q+W-1])
// All arithmetic is on fp32 pairs of adjacent channels (FFMA2: two FMAs per issue slot).
// `wy`, `bv` are the taps and bias scaled by ActGrad::kPre for the pre-activation, `wv` the taps
// divided by ActGrad::kGScale for dx; g (gc, gwin, and through it dw) carries the factor kGScale.
template <typename T, int W, int C, bool kSilu, bool kMask, bool kTanh>
__device__ __forceinline__ void bwd_cl_position_impl(
    const Raw<T, C> &xraw, const Raw<T, C> &draw, int sid, bool accumulate, bool store_dx, bool store_dinit,
    float2 (&xwin)[W - 1][C / 2], float2 (&gwin)[W - 1][C / 2], int (&swin)[W - 1], const float2 (&wv)[W][C / 2],
    const float2 (&wy)[W][C / 2], const float2 (&bv)[C / 2], float2 (&dw)[C / 2][W + 1], const T *dfin_ptr, int64_t df_cs,
    char *dx_ptr, T *dinit_ptr) {
    constexpr int P = C / 2;
    float2 xc[P], gc[P];
    unpack_pairs<T>(xraw, xc);
    unpack_pairs<T>(draw, gc);   // dout, turned into g below
    #pragma unroll
    for (int c = 0; c < P; ++c) {
        if (kSilu) {
            float2 y = bv[c];
            #pragma unroll
            for (int k = 0; k < W - 1; ++k) {
                if (!kMask || swin[k] == sid) y = fma2(wy[k][c], xwin[k][c], y);
            }
            y = fma2(wy[W - 1][c], xc[c], y);
            gc[c] = act_grad_pair<kTanh>(y, gc[c]);
        }
        if (kMask && sid < 0) gc[c] = make_float2(0.f, 0.f);   // padded token: out == 0 identically
    }
    if (accumulate) {
        #pragma unroll
        for (int c = 0; c < P; ++c) {
            dw[c][W] = add2(dw[c][W], gc[c]);
            #pragma unroll
            for (int k = 0; k < W - 1; ++k) {
                if (!kMask || swin[k] == sid) dw[c][k] = fma2(xwin[k][c], gc[c], dw[c][k]);
            }
            dw[c][W - 1] = fma2(xc[c], gc[c], dw[c][W - 1]);
        }
    }
    if (store_dx || store_dinit) {
        float2 o[P];
        #pragma unroll
        for (int c = 0; c < P; ++c) {
            float2 acc = make_float2(0.f, 0.f);
            #pragma unroll
            for (int m = 0; m < W - 1; ++m) {
                if (!kMask || swin[m] == swin[0]) acc = fma2(wv[W - 1 - m][c], gwin[m][c], acc);
            }
            if (!kMask || sid == swin[0]) acc = fma2(wv[0][c], gc[c], acc);
            o[c] = acc;
        }
        if (dfin_ptr != nullptr) {
            #pragma unroll
            for (int c = 0; c < P; ++c) {
                o[c].x += Elem<T>::to_f(dfin_ptr[(2 * c) * df_cs]);
                o[c].y += Elem<T>::to_f(dfin_ptr[(2 * c + 1) * df_cs]);
            }
        }
        if (store_dx) st_stream_raw(dx_ptr, PackPairs<T, C>::run(o));
        else st_plain_raw(dinit_ptr, PackPairs<T, C>::run(o));
    }
    #pragma unroll
    for (int k = 0; k < W - 2; ++k) {
        #pragma unroll
        for (int c = 0; c < P; ++c) { xwin[k][c] = xwin[k + 1][c]; gwin[k][c] = gwin[k + 1][c]; }
        if (kMask) swin[k] = swin[k + 1];
    }
    #pragma unroll
    for (int c = 0; c < P; ++c) { xwin[W - 2][c] = xc[c]; gwin[W - 2][c] = gc[c]; }
    // unmasked code only ever runs when every id in the window already equals sid (or there are no ids)
    if (kMask) swin[W - 2] = sid;
}

// seq_idx depends on (batch, token) only, so it is uniform across a warp.  Sequence
// boundaries are rare: when the window and the current token all carry one non-negative id,
// no tap is masked and the unmasked code runs (a warp-uniform branch).
template <typename T, int W, int C, bool kSilu, bool kSeqIdx, bool kTanh>
__device__ __forceinline__ void bwd_cl_position(
    const Raw<T, C> &xraw, const Raw<T, C> &draw, int sid, bool accumulate, bool store_dx, bool store_dinit,
    float2 (&xwin)[W - 1][C / 2], float2 (&gwin)[W - 1][C / 2], int (&swin)[W - 1], const float2 (&wv)[W][C / 2],
    const float2 (&wy)[W][C / 2], const float2 (&bv)[C / 2], float2 (&dw)[C / 2][W + 1], const T *dfin_ptr, int64_t df_cs,
    char *dx_ptr, T *dinit_ptr) {
    if (kSeqIdx) {
        bool same = sid >= 0;
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) same = same && swin[k] == sid;
        if (same) {
            bwd_cl_position_impl<T, W, C, kSilu, false, kTanh>(xraw, draw, sid, accumulate, store_dx, store_dinit, xwin, gwin,
                                                                 swin, wv, wy, bv, dw, dfin_ptr, df_cs, dx_ptr, dinit_ptr);
            return;
        }
    }
    bwd_cl_position_impl<T, W, C, kSilu, kSeqIdx, kTanh>(xraw, draw, sid, accumulate, store_dx, store_dinit, xwin, gwin, swin,
                                                           wv, wy, bv, dw, dfin_ptr, df_cs, dx_ptr, dinit_ptr);
}

template <typename T, int W, bool kSilu, bool kSeqIdx>
__global__ void __launch_bounds__(32 * kBwdClRows, CC1D_BWD_CL_MINBLK) bwd_cl_kernel(const BwdClArgs a) {
    pdl_wait();
    constexpr int C = kBwdClC;
    constexpr int U = kBwdClUnroll;
    constexpr int kAcc = (W + 1) * C;                    // fp32 partial sums per thread
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
    using R = Raw<T, C>;
    __shared__ __align__(16) float s_red[(kBwdClRows - 1) * 32 * kAcc];

    const uint32_t cb = blockIdx.x % a.ncolblk;
    const uint32_t rest = blockIdx.x / a.ncolblk;
    const uint32_t grp = rest % a.ngroups;
    const uint32_t b = rest / a.ngroups;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const uint32_t col = cb * 32 + tx;
    const int L = (int)a.seqlen;
    const int t0 = (int)((grp * kBwdClRows + ty) * (uint32_t)a.tpt);
    const bool active = col < a.ncols && t0 < L;

    float2 dw[C / 2][W + 1];   // pairs of adjacent channels; [.][W] is dbias
    #pragma unroll
    for (int c = 0; c < C / 2; ++c) {
        #pragma unroll
        for (int k = 0; k <= W; ++k) dw[c][k] = make_float2(0.f, 0.f);
    }

    if (active) {
        const int t1 = t0 + a.tpt < L ? t0 + a.tpt : L;
        const int n_ext = t1 - t0 + (W - 1);                                   // positions to process
        const int n_ld = (t1 + (W - 1) < L ? t1 + (W - 1) : L) - t0;            // positions that exist
        const int n_x = kSilu ? n_ld : t1 - t0;                                 // x past the chunk only feeds y
        const int64_t xs = a.x_ls * (int64_t)sizeof(T), ds = a.d_ls * (int64_t)sizeof(T), os = a.o_ls * (int64_t)sizeof(T);
        const int64_t cofs = (int64_t)col * C * (int64_t)sizeof(T);
        const char *xptr = reinterpret_cast<const char *>(a.x) + b * a.x_bs * (int64_t)sizeof(T) + cofs + t0 * xs;
        const char *dptr = reinterpret_cast<const char *>(a.dout) + b * a.d_bs * (int64_t)sizeof(T) + cofs + t0 * ds;
        char *optr = reinterpret_cast<char *>(a.dx) + b * a.o_bs * (int64_t)sizeof(T) + cofs + (t0 - (W - 1)) * os;
        const int32_t *__restrict__ sp = kSeqIdx ? a.seq_idx + (int64_t)b * L + t0 : nullptr;

        R xr[U], dr[U];
        int sid[U];
        #pragma unroll
        for (int u = 0; u < U; ++u) {
            zero_raw(xr[u]); zero_raw(dr[u]);
            sid[u] = -2;   // beyond the sequence: matches nothing
            if (u < n_x) ld_stream_raw(xr[u], xptr + u * xs);
            if (u < n_ld) {
                ld_stream_raw(dr[u], dptr + u * ds);
                if (kSeqIdx) sid[u] = sp[u];
            }
        }
        // x at the width-1 positions before t0 (x, initial_states or zero); g before t0 is never used
        float2 xwin[W - 1][C / 2], gwin[W - 1][C / 2];
        int swin[W - 1];
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) {
            const int p = t0 - (W - 1) + k;
            R r;
            zero_raw(r);
            swin[k] = -1;
            if (p >= 0) {
                ld_cached_raw(r, xptr - (W - 1 - k) * xs);
                if (kSeqIdx) swin[k] = sp[k - (W - 1)];
            } else if (a.init != nullptr) {
                ld_cached_raw(r, reinterpret_cast<const T *>(a.init) + b * a.i_bs + (p + (W - 1)) * a.i_ls + (int64_t)col * C);
            }
            unpack_pairs<T>(r, xwin[k]);
            #pragma unroll
            for (int c = 0; c < C / 2; ++c) gwin[k][c] = make_float2(0.f, 0.f);
        }
        float2 wv[W][C / 2], wy[W][C / 2], bv[C / 2];
        load_taps_pairs<W, C>(wv, bv, a.weight, a.w_cs, a.w_ws, a.bias, a.wtype, (int64_t)col * C, 1.f);
        scale_taps_for_backward<W, C, kTanh>(wv, wy, bv);

        const bool want_dinit = a.dinit != nullptr && t0 == 0;
        const T *dfin_base = a.dfin != nullptr ? reinterpret_cast<const T *>(a.dfin) + b * a.df_bs + (int64_t)col * C * a.df_cs : nullptr;
        T *dinit_base = want_dinit ? reinterpret_cast<T *>(a.dinit) + b * a.di_bs + (int64_t)col * C : nullptr;

        // Positions are processed in blocks of U with the next block's loads in flight.  Blocks
        // that lie fully inside [t0 + W-1, t1) take the unconditional path (every position both
        // accumulates and stores dx), so the window rotation stays in renamed registers; the
        // first block and the blocks around the chunk end take the flagged path.
        const int n_in = t1 - t0;
        for (int base = 0; base < n_ext; base += U) {
            R xn[U], dn[U];
            int nsid[U];
            #pragma unroll
            for (int u = 0; u < U; ++u) {
                zero_raw(xn[u]); zero_raw(dn[u]);
                nsid[u] = -2;
                const int i = base + U + u;
                if (i < n_x) ld_stream_raw(xn[u], xptr + (U + u) * xs);
                if (i < n_ld) {
                    ld_stream_raw(dn[u], dptr + (U + u) * ds);
                    if (kSeqIdx) nsid[u] = sp[U + u];
                }
            }
            const bool steady = base >= W - 1 && base + U <= n_in && (a.dfin == nullptr || t0 + base + U <= L - (W - 1));
            if (steady) {
                #pragma unroll
                for (int u = 0; u < U; ++u) {
                    bwd_cl_position<T, W, C, kSilu, kSeqIdx, kTanh>(
                        xr[u], dr[u], sid[u], true, true, false, xwin, gwin, swin, wv, wy, bv, dw, nullptr, 0,
                        optr + u * os, nullptr);
                }
            } else {
                #pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int i = base + u;          // position t0 + i
                    if (i < n_ext) {
                        const int q = t0 + i - (W - 1);   // dx position produced now
                        const bool st_dx = i >= W - 1;     // q >= t0 (q < t1 always holds)
                        const bool st_di = q < 0 && want_dinit;
                        const T *df = (dfin_base != nullptr && q >= L - (W - 1)) ? dfin_base + (q - (L - (W - 1))) * a.df_ls : nullptr;
                        T *di = st_di ? dinit_base + (q + (W - 1)) * a.di_ls : nullptr;
                        bwd_cl_position<T, W, C, kSilu, kSeqIdx, kTanh>(
                            xr[u], dr[u], sid[u], i < n_in, st_dx, st_di, xwin, gwin, swin, wv, wy, bv, dw, df, a.df_cs,
                            optr + u * os, di);
                    }
                }
            }
            xptr += U * xs; dptr += U * ds; optr += U * os;
            if (kSeqIdx) sp += U;
            #pragma unroll
            for (int u = 0; u < U; ++u) { xr[u] = xn[u]; dr[u] = dn[u]; sid[u] = nsid[u]; }
        }
    }

    // fixed-order sum over the CTA's token chunks: rows 1..7 park their sums, row 0 adds them
    // in ascending row order and writes the CTA's partial row
    // channel c of the thread lives in pair c/2, component c%2
    auto dwv = [&](int c, int k) -> float & { return (c & 1) ? dw[c >> 1][k].y : dw[c >> 1][k].x; };
    unscale_sums<W, C, kTanh>(dw);
    if (ty > 0) {
        float *r = s_red + ((ty - 1) * 32 + tx) * kAcc;
        #pragma unroll
        for (int c = 0; c < C; ++c) {
            #pragma unroll
            for (int k = 0; k <= W; ++k) r[c * (W + 1) + k] = dwv(c, k);
        }
    }
    __syncthreads();
    if (ty == 0 && col < a.ncols) {
        #pragma unroll 1
        for (int y = 1; y < kBwdClRows; ++y) {
            const float *r = s_red + ((y - 1) * 32 + tx) * kAcc;
            #pragma unroll
            for (int c = 0; c < C; ++c) {
                #pragma unroll
                for (int k = 0; k <= W; ++k) dwv(c, k) += r[c * (W + 1) + k];
            }
        }
        float *p = a.ws + (((uint64_t)b * a.ngroups + grp) * (uint64_t)a.dim + (uint64_t)col * C) * (W + 1);
        #pragma unroll
        for (int c = 0; c < C; ++c) {
            #pragma unroll
            for (int k = 0; k <= W; ++k) p[c * (W + 1) + k] = dwv(c, k);
        }
    }
}

// ---- TMA variant ----------------------------------------------------------------------------
// Same arithmetic and the same partial-row layout as bwd_cl_kernel, but x and dout reach the
// warp through the TMA unit: each warp is an independent pipeline over its own ring of
// kBwdTmaStages stages, a stage = one x box + one dout box of [kTmaRows positions x 32 lanes x
// C channels], one mbarrier per stage.  Rows past seqlen arrive as zeros, which is exactly what
// the right halo needs (x = 0, dout = 0 beyond the sequence).
#ifndef CC1D_BWD_CL_TMA
#define CC1D_BWD_CL_TMA 1
#endif
#ifndef CC1D_BWD_TMA_STAGES
#define CC1D_BWD_TMA_STAGES 3
#endif
constexpr int kBwdTmaStages = CC1D_BWD_TMA_STAGES;

template <typename T> struct BwdTma {
    static constexpr int kRowBytes = 32 * kBwdClC * (int)sizeof(T);      // one token of a warp's strip
    static constexpr int kBoxBytes = kTmaRows * kRowBytes;
    static constexpr int kStageBytes = 2 * kBoxBytes;                     // x box, then dout box
    static constexpr size_t kSmem = (size_t)kBwdClRows * kBwdTmaStages * kStageBytes + (size_t)kBwdClRows * kBwdTmaStages * 8;
};

template <typename R> __device__ __forceinline__ R lds_raw(uint32_t addr);
template <> __device__ __forceinline__ uint4 lds_raw<uint4>(uint32_t addr) { return lds128(addr); }
template <> __device__ __forceinline__ uint2 lds_raw<uint2>(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// kDoutCf: dout is stored channel-first ((batch, dim, seqlen) with seqlen stride 1) although x and dx are
// channel-last: its box arrives as [32 * C channels][kTmaRows tokens] (16 bytes per channel), a thread
// reads the C rows of its channels once per stage and picks token r out of them with byte permutes.
template <typename T, int W, bool kSilu, bool kSeqIdx, bool kDoutCf>
__global__ void __launch_bounds__(32 * kBwdClRows, CC1D_BWD_CL_MINBLK)
bwd_cl_tma_kernel(const BwdClArgs a, const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap dmap) {
    pdl_wait();
    constexpr int C = kBwdClC;
    constexpr int kAcc = (W + 1) * C;
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
    constexpr int kRowBytes = BwdTma<T>::kRowBytes, kBoxBytes = BwdTma<T>::kBoxBytes, kStageBytes = BwdTma<T>::kStageBytes;
    using R = Raw<T, C>;
    __shared__ __align__(16) float s_red[(kBwdClRows - 1) * 32 * kAcc];
    extern __shared__ __align__(1024) unsigned char smem[];

    const uint32_t cb = blockIdx.x % a.ncolblk;
    const uint32_t rest = blockIdx.x / a.ncolblk;
    const uint32_t grp = rest % a.ngroups;
    const uint32_t b = rest / a.ngroups;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const uint32_t col = cb * 32 + tx;
    const bool lane_ok = col < a.ncols;
    const int L = (int)a.seqlen;
    const int t0 = (int)((grp * kBwdClRows + ty) * (uint32_t)a.tpt);
    const bool active = t0 < L;                      // warp-uniform

    float2 dw[C / 2][W + 1];   // pairs of adjacent channels; [.][W] is dbias
    #pragma unroll
    for (int c = 0; c < C / 2; ++c) {
        #pragma unroll
        for (int k = 0; k <= W; ++k) dw[c][k] = make_float2(0.f, 0.f);
    }

    if (active) {
        const int t1 = t0 + a.tpt < L ? t0 + a.tpt : L;
        const int n_in = t1 - t0;
        const int n_ext = n_in + (W - 1);                 // positions to process
        const int nst = (n_ext + kTmaRows - 1) / kTmaRows;
        const uint32_t ring = smem_u32(smem) + ty * (kBwdTmaStages * kStageBytes);
        const uint32_t bars = smem_u32(smem) + kBwdClRows * kBwdTmaStages * kStageBytes + ty * (kBwdTmaStages * 8);
        const int c0 = (int)(cb * 32 * C);
        if (tx == 0) {
            tma_prefetch_desc(&xmap);
            tma_prefetch_desc(&dmap);
            #pragma unroll
            for (int s = 0; s < kBwdTmaStages; ++s) mbar_init(bars + 8 * s, 1);
            fence_mbar_init();
            #pragma unroll
            for (int s = 0; s < kBwdTmaStages; ++s) {
                if (s < nst) {
                    mbar_expect_tx(bars + 8 * s, kStageBytes);
                    tma_load_3d(ring + s * kStageBytes, &xmap, c0, t0 + s * kTmaRows, (int)b, bars + 8 * s);
                    if (kDoutCf) tma_load_3d(ring + s * kStageBytes + kBoxBytes, &dmap, t0 + s * kTmaRows, c0, (int)b, bars + 8 * s);
                    else tma_load_3d(ring + s * kStageBytes + kBoxBytes, &dmap, c0, t0 + s * kTmaRows, (int)b, bars + 8 * s);
                }
            }
        }
        __syncwarp();

        const int64_t xs = a.x_ls * (int64_t)sizeof(T), os = a.o_ls * (int64_t)sizeof(T);
        const int64_t cofs = (int64_t)col * C * (int64_t)sizeof(T);
        const char *xptr = reinterpret_cast<const char *>(a.x) + b * a.x_bs * (int64_t)sizeof(T) + cofs + t0 * xs;
        char *optr = reinterpret_cast<char *>(a.dx) + b * a.o_bs * (int64_t)sizeof(T) + cofs + (t0 - (W - 1)) * os;
        const int32_t *__restrict__ sp = kSeqIdx ? a.seq_idx + (int64_t)b * L + t0 : nullptr;
        const int n_ld = (t1 + (W - 1) < L ? t1 + (W - 1) : L) - t0;   // positions that exist

        // x at the width-1 positions before t0 (x, initial_states or zero); g before t0 is never used
        float2 xwin[W - 1][C / 2], gwin[W - 1][C / 2];
        int swin[W - 1];
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) {
            const int p = t0 - (W - 1) + k;
            R r;
            zero_raw(r);
            swin[k] = -1;
            if (p >= 0) {
                if (lane_ok) ld_cached_raw(r, xptr - (W - 1 - k) * xs);
                if (kSeqIdx) swin[k] = sp[k - (W - 1)];
            } else if (a.init != nullptr && lane_ok) {
                ld_cached_raw(r, reinterpret_cast<const T *>(a.init) + b * a.i_bs + (p + (W - 1)) * a.i_ls + (int64_t)col * C);
            }
            unpack_pairs<T>(r, xwin[k]);
            #pragma unroll
            for (int c = 0; c < C / 2; ++c) gwin[k][c] = make_float2(0.f, 0.f);
        }
        float2 wv[W][C / 2], wy[W][C / 2], bv[C / 2];
        if (lane_ok) {
            load_taps_pairs<W, C>(wv, bv, a.weight, a.w_cs, a.w_ws, a.bias, a.wtype, (int64_t)col * C, 1.f);
        } else {
            #pragma unroll
            for (int c = 0; c < C / 2; ++c) {
                bv[c] = make_float2(0.f, 0.f);
                #pragma unroll
                for (int k = 0; k < W; ++k) wv[k][c] = make_float2(0.f, 0.f);
            }
        }
        scale_taps_for_backward<W, C, kTanh>(wv, wy, bv);
        const bool want_dinit = a.dinit != nullptr && t0 == 0 && lane_ok;
        const T *dfin_base = (a.dfin != nullptr && lane_ok) ? reinterpret_cast<const T *>(a.dfin) + b * a.df_bs + (int64_t)col * C * a.df_cs : nullptr;
        T *dinit_base = want_dinit ? reinterpret_cast<T *>(a.dinit) + b * a.di_bs + (int64_t)col * C : nullptr;

        // sequence ids one stage ahead, one per lane: lane l holds the id of row l % kTmaRows of the
        // stage; -2 beyond the sequence (matches nothing)
        const int myrow = tx & (kTmaRows - 1);
        int next_id = (kSeqIdx && myrow < n_ld) ? sp[myrow] : -2;

        for (int st = 0; st < nst; ++st) {
            const int s = st % kBwdTmaStages;
            const int base = st * kTmaRows;
            const int my_id = next_id;
            next_id = (kSeqIdx && base + kTmaRows + myrow < n_ld) ? sp[kTmaRows + myrow] : -2;
            // the warp decides together (the votes and shuffles below need all 32 lanes)
            if (!__all_sync(kFullMask, mbar_wait(bars + 8 * s, (uint32_t)(st / kBwdTmaStages) & 1u))) {
                g_tma_wait_expired = 1;     // never expected; stop consuming, still join the block reduction
                break;
            }
            const uint32_t xsrc = ring + s * kStageBytes + tx * (C * (int)sizeof(T));
            const uint32_t dsrc = xsrc + kBoxBytes;
            // channel-first dout: the thread's C channel rows of this stage, kTmaRows tokens each
            uint4 dch[C];
            if (kDoutCf) {
                #pragma unroll
                for (int j = 0; j < C; ++j) dch[j] = lds128(ring + s * kStageBytes + kBoxBytes + (tx * C + j) * 16);
            }
            auto dout_row = [&](int r) -> R {
                if constexpr (kDoutCf) {
                    static_assert(!kDoutCf || (sizeof(T) == 2 && C == 4), "channel-first dout: 16-bit types, 4 channels per thread");
                    const uint32_t w0 = (r >> 1) == 0 ? dch[0].x : (r >> 1) == 1 ? dch[0].y : (r >> 1) == 2 ? dch[0].z : dch[0].w;
                    const uint32_t w1 = (r >> 1) == 0 ? dch[1].x : (r >> 1) == 1 ? dch[1].y : (r >> 1) == 2 ? dch[1].z : dch[1].w;
                    const uint32_t w2 = (r >> 1) == 0 ? dch[2].x : (r >> 1) == 1 ? dch[2].y : (r >> 1) == 2 ? dch[2].z : dch[2].w;
                    const uint32_t w3 = (r >> 1) == 0 ? dch[3].x : (r >> 1) == 1 ? dch[3].y : (r >> 1) == 2 ? dch[3].z : dch[3].w;
                    const uint32_t sel = (r & 1) ? 0x7632u : 0x5410u;
                    R v;
                    v.x = __byte_perm(w0, w1, sel);
                    v.y = __byte_perm(w2, w3, sel);
                    return v;
                } else {
                    return lds_raw<R>(dsrc + r * kRowBytes);
                }
            };
            const bool steady = base >= W - 1 && base + kTmaRows <= n_in &&
                                (a.dfin == nullptr || t0 + base + kTmaRows <= L - (W - 1));
            // one test per stage instead of one per position: when the window and all positions of
            // the stage carry the same non-negative sequence id, nothing is masked (warp-uniform)
            bool plain = steady;
            if (kSeqIdx) {
                const int first = __shfl_sync(kFullMask, my_id, 0);
                bool same = my_id == first && first >= 0;
                #pragma unroll
                for (int k = 0; k < W - 1; ++k) same = same && swin[k] == first;
                plain = __all_sync(kFullMask, same) && plain;
            }
            if (plain) {
                #pragma unroll
                for (int r = 0; r < kTmaRows; ++r) {
                    const R xr = lds_raw<R>(xsrc + r * kRowBytes), dr = dout_row(r);
                    bwd_cl_position_impl<T, W, C, kSilu, false, kTanh>(
                        xr, dr, 0, true, lane_ok, false, xwin, gwin, swin, wv, wy, bv, dw, nullptr, 0, optr + r * os, nullptr);
                }
            } else if (steady) {
                // a stage that holds a sequence boundary: rare, so kept compact (not unrolled) -- the
                // kernel's code size is what the steady-state loop above pays for in instruction fetches
                #pragma unroll 1
                for (int r = 0; r < kTmaRows; ++r) {
                    const int sid = kSeqIdx ? __shfl_sync(kFullMask, my_id, r) : 0;
                    const R xr = lds_raw<R>(xsrc + r * kRowBytes), dr = dout_row(r);
                    bwd_cl_position_impl<T, W, C, kSilu, kSeqIdx, kTanh>(
                        xr, dr, sid, true, lane_ok, false, xwin, gwin, swin, wv, wy, bv, dw, nullptr, 0, optr + r * os, nullptr);
                }
            } else {
                #pragma unroll
                for (int r = 0; r < kTmaRows; ++r) {
                    const int i = base + r;               // position t0 + i
                    const int sid = kSeqIdx ? __shfl_sync(kFullMask, my_id, r) : 0;
                    if (i < n_ext) {
                        const R xr = lds_raw<R>(xsrc + r * kRowBytes), dr = dout_row(r);
                        const int q = t0 + i - (W - 1);   // dx position produced now
                        const bool st_dx = i >= W - 1 && lane_ok;
                        const bool st_di = q < 0 && want_dinit;
                        const T *df = (dfin_base != nullptr && q >= L - (W - 1)) ? dfin_base + (q - (L - (W - 1))) * a.df_ls : nullptr;
                        T *di = st_di ? dinit_base + (q + (W - 1)) * a.di_ls : nullptr;
                        bwd_cl_position<T, W, C, kSilu, kSeqIdx, kTanh>(
                            xr, dr, sid, i < n_in, st_dx, st_di, xwin, gwin, swin, wv, wy, bv, dw, df, a.df_cs, optr + r * os, di);
                    }
                }
            }
            optr += kTmaRows * os;
            if (kSeqIdx) sp += kTmaRows;
            __syncwarp();                                   // every lane has consumed the stage
            if (tx == 0 && st + kBwdTmaStages < nst) {      // refill it
                fence_proxy_async_smem();
                mbar_expect_tx(bars + 8 * s, kStageBytes);
                tma_load_3d(ring + s * kStageBytes, &xmap, c0, t0 + (st + kBwdTmaStages) * kTmaRows, (int)b, bars + 8 * s);
                if (kDoutCf) tma_load_3d(ring + s * kStageBytes + kBoxBytes, &dmap, t0 + (st + kBwdTmaStages) * kTmaRows, c0, (int)b, bars + 8 * s);
                else tma_load_3d(ring + s * kStageBytes + kBoxBytes, &dmap, c0, t0 + (st + kBwdTmaStages) * kTmaRows, (int)b, bars + 8 * s);
            }
        }
    }

    // fixed-order sum over the CTA's token chunks (see bwd_cl_kernel)
    auto dwv = [&](int c, int k) -> float & { return (c & 1) ? dw[c >> 1][k].y : dw[c >> 1][k].x; };
    unscale_sums<W, C, kTanh>(dw);
    if (ty > 0) {
        float *r = s_red + ((ty - 1) * 32 + tx) * kAcc;
        #pragma unroll
        for (int c = 0; c < C; ++c) {
            #pragma unroll
            for (int k = 0; k <= W; ++k) r[c * (W + 1) + k] = dwv(c, k);
        }
    }
    __syncthreads();
    if (ty == 0 && lane_ok) {
        #pragma unroll 1
        for (int y = 1; y < kBwdClRows; ++y) {
            const float *r = s_red + ((y - 1) * 32 + tx) * kAcc;
            #pragma unroll
            for (int c = 0; c < C; ++c) {
                #pragma unroll
                for (int k = 0; k <= W; ++k) dwv(c, k) += r[c * (W + 1) + k];
            }
        }
        float *p = a.ws + (((uint64_t)b * a.ngroups + grp) * (uint64_t)a.dim + (uint64_t)col * C) * (W + 1);
        #pragma unroll
        for (int c = 0; c < C; ++c) {
            #pragma unroll
            for (int k = 0; k <= W; ++k) p[c * (W + 1) + k] = dwv(c, k);
        }
    }
}

int pick_tokens_per_thread(int64_t batch, int64_t ncols, int64_t seqlen, int sms, int max_tpt);
int pick_chunk_tokens(int64_t batch, int64_t ncolblk, int64_t seqlen, int warps_per_cta, int64_t resident_ctas,
                      const int *candidates, int n, int overhead);

struct ClPlan {
    int tpt;
    uint32_t ncols, ncolblk, ngroups;
};

static ClPlan plan_channel_last(const cc1d_bwd_params &p) {
    const int C = kBwdClC;
    ClPlan pl;
    const int64_t ncols = p.dim / C;
    pl.tpt = pick_tokens_per_thread(p.batch, ncols, p.seqlen, kTilingSMs / 2, 128);
    pl.ncols = (uint32_t)ncols;
    pl.ncolblk = (uint32_t)((ncols + 31) / 32);
    if (pl.tpt == 128 && p.itype != CC1D_F32) {
        // 16-bit (TMA) kernel on a problem of several waves: pick the chunk length by the waves it makes.
        // Measured, bf16: (1,5376,32768) 128 tokens (6.05 waves) 204 us, 160 tokens (4.9 waves) 196 us;
        // (8,5120,2048) 128 tokens (2.9 waves) 103 us, 160 tokens 116 us.  Multiples of 8 tokens: a
        // channel-first dout box starts at the chunk's first token.
        static const int kChunks[] = {128, 160, 192};
        pl.tpt = pick_chunk_tokens(p.batch, pl.ncolblk, p.seqlen, kBwdClRows, (int64_t)kTilingSMs * CC1D_BWD_CL_MINBLK, kChunks, 3, 16);
    }
    const int64_t chunks = (p.seqlen + pl.tpt - 1) / pl.tpt;
    pl.ngroups = (uint32_t)((chunks + kBwdClRows - 1) / kBwdClRows);
    return pl;
}

size_t bwd_workspace_bytes_channel_last(const cc1d_bwd_params &p) {
    const ClPlan pl = plan_channel_last(p);
    return (size_t)((uint64_t)p.batch * pl.ngroups * (uint64_t)p.dim * (uint64_t)(p.width + 1) * sizeof(float));
}

int launch_bwd_channel_last(const cc1d_bwd_params &p, cudaStream_t stream) {
    const int C = kBwdClC;
    // token positions are 32-bit integers in the kernels (chunk starts plus a halo must not wrap)
    if (p.seqlen >= (1ll << 31) - 4096 || p.dim >= (1ll << 31)) return CC1D_ERR_TOO_LARGE;
    if (!is_aligned16(p.x) || !is_aligned16(p.dout) || !is_aligned16(p.dx)) return CC1D_ERR_ALIGN;
    if (p.initial_states && (!is_aligned16(p.initial_states) || p.initial_states_batch_stride % C ||
                             p.initial_states_l_stride % C)) return CC1D_ERR_ALIGN;
    if (p.dinitial_states && (!is_aligned16(p.dinitial_states) || p.dinitial_states_batch_stride % C ||
                              p.dinitial_states_l_stride % C)) return CC1D_ERR_ALIGN;
    const ClPlan pl = plan_channel_last(p);
    // dout stored channel-first beside a channel-last x (what autograd hands over when the consumer of
    // `out` made it contiguous): read in place through a second kind of tensor map, no re-layout copy
    const bool dout_cf = p.seqlen > 1 && p.dim > 1 && p.dout_l_stride == 1 && p.dout_c_stride != 1;
    const uint64_t ctas = (uint64_t)pl.ncolblk * pl.ngroups * (uint64_t)p.batch;
    if (ctas >= (1ull << 31)) return CC1D_ERR_TOO_LARGE;
    if (bwd_workspace_bytes_channel_last(p) > p.workspace_bytes) return CC1D_ERR_WORKSPACE;
    if (!is_aligned16(p.workspace)) return CC1D_ERR_ALIGN;

    BwdClArgs a;
    a.x = p.x; a.dout = p.dout; a.dx = p.dx; a.weight = p.weight; a.bias = p.bias; a.seq_idx = p.seq_idx;
    a.init = p.initial_states; a.dfin = p.dfinal_states; a.dinit = p.dinitial_states;
    a.ws = reinterpret_cast<float *>(p.workspace);
    a.x_bs = p.x_batch_stride; a.x_ls = p.x_l_stride; a.d_bs = p.dout_batch_stride; a.d_ls = p.dout_l_stride;
    a.o_bs = p.dx_batch_stride; a.o_ls = p.dx_l_stride; a.w_cs = p.weight_c_stride; a.w_ws = p.weight_width_stride;
    a.i_bs = p.initial_states_batch_stride; a.i_ls = p.initial_states_l_stride;
    a.df_bs = p.dfinal_states_batch_stride; a.df_cs = p.dfinal_states_c_stride; a.df_ls = p.dfinal_states_l_stride;
    a.di_bs = p.dinitial_states_batch_stride; a.di_ls = p.dinitial_states_l_stride;
    a.dim = p.dim; a.seqlen = p.seqlen; a.wtype = p.wtype; a.tpt = pl.tpt;
    a.ncols = pl.ncols; a.ncolblk = pl.ncolblk; a.ngroups = pl.ngroups;
    if (ctas > 0 && p.phase != 2) {
        bool launched = false;
#if CC1D_BWD_CL_TMA
        CUtensorMap xmap, dmap;
        const int row_bytes = 32 * kBwdClC * elem_size(p.itype);
        // fp32 stages are twice as large (2 CTAs per SM instead of 3): still 3 % ahead of the register-prefetch
        // kernel; a channel-first dout is read in place for 16-bit types only
        if ((p.itype != CC1D_F32 || !dout_cf) && p.seqlen < (1ll << 31) - 16 && p.batch < (1ll << 31) &&
            make_channel_last_tensor_map(&xmap, p.itype, p.x, p.dim, p.seqlen, p.batch, p.x_l_stride, p.x_batch_stride, row_bytes) &&
            (dout_cf ? make_channel_first_tensor_map(&dmap, p.itype, p.dout, p.seqlen, p.dim, p.batch, p.dout_c_stride,
                                                     p.dout_batch_stride, kTmaRows, 32 * kBwdClC)
                     : make_channel_last_tensor_map(&dmap, p.itype, p.dout, p.dim, p.seqlen, p.batch, p.dout_l_stride,
                                                    p.dout_batch_stride, row_bytes))) {
            if (p.itype == CC1D_F32) {
                using T = float;
                CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu, CC1D_DISPATCH_BOOL(p.seq_idx != nullptr, kSeqIdx, {
                        auto kernel = bwd_cl_tma_kernel<T, W, kSilu, kSeqIdx, false>;
                        allow_dynamic_smem(reinterpret_cast<const void *>(kernel), BwdTma<T>::kSmem);
                        launch_k(kernel, dim3((unsigned)ctas), dim3(32 * kBwdClRows), BwdTma<T>::kSmem, stream, a, xmap, dmap);
                    });););
            } else if (p.itype == CC1D_BF16) {
                using T = __nv_bfloat16;
                CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu, CC1D_DISPATCH_BOOL(p.seq_idx != nullptr, kSeqIdx,
                    CC1D_DISPATCH_BOOL(dout_cf, kDoutCf, {
                        auto kernel = bwd_cl_tma_kernel<T, W, kSilu, kSeqIdx, kDoutCf>;
                        allow_dynamic_smem(reinterpret_cast<const void *>(kernel), BwdTma<T>::kSmem);
                        launch_k(kernel, dim3((unsigned)ctas), dim3(32 * kBwdClRows), BwdTma<T>::kSmem, stream, a, xmap, dmap);
                    }););););
            } else {
                using T = __half;
                CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu, CC1D_DISPATCH_BOOL(p.seq_idx != nullptr, kSeqIdx,
                    CC1D_DISPATCH_BOOL(dout_cf, kDoutCf, {
                        auto kernel = bwd_cl_tma_kernel<T, W, kSilu, kSeqIdx, kDoutCf>;
                        allow_dynamic_smem(reinterpret_cast<const void *>(kernel), BwdTma<T>::kSmem);
                        launch_k(kernel, dim3((unsigned)ctas), dim3(32 * kBwdClRows), BwdTma<T>::kSmem, stream, a, xmap, dmap);
                    }););););
            }
            launched = true;
        }
#endif
        // a channel-first dout is only served by the TMA kernel (16-bit types, a tensor map the driver accepts)
        if (!launched && dout_cf) return CC1D_ERR_STRIDE;
        if (!launched) {
            CC1D_DISPATCH_ITYPE(p.itype, CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu,
                CC1D_DISPATCH_BOOL(p.seq_idx != nullptr, kSeqIdx, {
                    launch_k(bwd_cl_kernel<T, W, kSilu, kSeqIdx>, dim3((unsigned)ctas), dim3(32 * kBwdClRows), 0, stream, a);
                }););););
        }
        if (check_launch() != CC1D_OK) return CC1D_ERR_LAUNCH;
    }
    ReduceArgs r;
    r.ws = a.ws; r.dweight = p.dweight; r.dbias = p.dbias;
    r.dw_cs = p.dweight_c_stride; r.dw_ws = p.dweight_width_stride;
    r.dim = p.dim;
    r.n_outer = (int64_t)p.batch * pl.ngroups;
    r.outer_stride = p.dim * (p.width + 1);
    r.n_inner = 1; r.inner_stride = 0;
    r.chan_stride = p.width + 1;
    r.accumulate = p.accumulate;
    set_peers(r, p.peers);
    if (p.dim == 0 || p.phase == 1) return CC1D_OK;
    if (p.seqlen == 0) r.n_outer = 0;
    return launch_reduce(r, p.width, stream);
}

int bwd_wait_expired() { return read_and_clear_wait_expired(); }

}  // namespace cc1d
