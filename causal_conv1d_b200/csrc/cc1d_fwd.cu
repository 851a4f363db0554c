// Forward kernels (sm_100a).
//
// Channel-first (x[b, c, :] contiguous): the work is cut into warp units of 32 * kVecs
// consecutive 16-byte vectors of one row.  A lane owns vector (j * 32 + lane); the
// (width-1)-element halo comes from the neighbouring lane by warp shuffle, only lane 0 of a
// unit's first vector re-reads one vector from global.  No shared memory, no barrier, every
// x byte is requested from DRAM once.  16-bit rows of a multiple of 16 elements on 32-byte
// aligned rows take fwd_cf_wide_kernel: 32 bytes per lane (256-bit loads and stores),
// arithmetic on fp32 pairs, half of the halos inside the lane.
//
// Channel-last (x[b, :, t] contiguous): a thread owns 4 adjacent channels (TMA kernel; one 16-byte
// vector in the kernel kept for tensors without a tensor map) and slides down `tpt` consecutive
// tokens keeping the last width-1 vectors in registers; a warp covers 128 channels of one token.
// seq_idx masking, initial_states (halo of the first chunk) and final_states (the window left
// after the last token) ride along.
//
// Replaces csrc/causal_conv1d_fwd.cu:46-137 (channel-first) and :205-348 (channel-last)
// of the reference.
#include "cc1d_common.cuh"
#include "cc1d_kernels.h"
#include "cc1d_tma.cuh"

namespace cc1d {

// ======================================================================================
// channel-first
// ======================================================================================
struct FwdCfArgs {
    const void *x;
    void *out;
    const void *weight;
    const void *bias;
    int64_t x_bs, x_cs, o_bs, o_cs, w_cs, w_ws;
    uint32_t dim, seqlen;
    int wtype;
    uint32_t vpr;      // 16-byte vectors per row, the last one may be partial
    uint32_t gpr;      // groups (32 * kVecs vectors) per row
    uint32_t gpu;      // groups per warp unit
    uint32_t upr;      // warp units per row
    uint32_t n_units;  // rows * upr
};

// A warp unit is `gpu` consecutive groups of 32 * kVecs vectors of one row, walked front to
// back: row decode and taps are paid once per unit, the halo of every group after the first
// is the previous group's last vector (still in lane 31's registers), and the next group's
// loads are issued before the current group is computed.
// kFull: seqlen is a multiple of the vector width and every group has all 32 * kVecs vectors,
// so no bounds check survives in the loop.
template <typename T, int W, bool kSilu, bool kFull, int kVecs>
__global__ void __launch_bounds__(256) fwd_cf_vec_kernel(const FwdCfArgs a) {
    pdl_wait();
    constexpr int V = Elem<T>::kVec;
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
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
        T *__restrict__ outr = reinterpret_cast<T *>(a.out) + b * a.o_bs + c * a.o_cs;
        const uint32_t g0 = seg * a.gpu;                                  // first group of the unit
        const uint32_t g1 = g0 + a.gpu < a.gpr ? g0 + a.gpu : a.gpr;      // one past the last
        uint32_t e0 = (g0 * (32 * kVecs) + lane) * V;                     // this lane's first element

        uint4 nxt[kVecs];
        #pragma unroll
        for (int j = 0; j < kVecs; ++j) nxt[j] = load_row_vec<T, kFull>(xr, e0 + j * 32 * V, L);
        uint4 carry = make_uint4(0, 0, 0, 0);   // vector that precedes this lane's first one
        if (lane == 31 && g0 > 0) carry = ld_cached(xr + (e0 - 32 * V));  // = vector before lane 0's

        // tanh form of SiLU works on y/2: fold the 1/2 into the taps
        const float pre = kTanh ? 0.5f : 1.f;
        float wv[W];
        #pragma unroll
        for (int k = 0; k < W; ++k) wv[k] = pre * load_w(a.weight, c * a.w_cs + k * a.w_ws, a.wtype);
        const float bv = a.bias != nullptr ? pre * load_w(a.bias, c, a.wtype) : 0.f;

        for (uint32_t g = g0; g < g1; ++g, e0 += kGroupElems) {
            uint4 raw[kVecs];
            #pragma unroll
            for (int j = 0; j < kVecs; ++j) raw[j] = nxt[j];
            if (g + 1 < g1) {
                #pragma unroll
                for (int j = 0; j < kVecs; ++j) nxt[j] = load_row_vec<T, kFull>(xr, e0 + kGroupElems + j * 32 * V, L);
            }
            #pragma unroll
            for (int j = 0; j < kVecs; ++j) {
                const uint4 prev = prev_vector_tail<V, W>(raw[j], j > 0 ? raw[j - 1] : carry, lane);
                const uint32_t e = e0 + j * 32 * V;
                if (!kFull && e >= L) continue;
                float xx[W - 1 + V];
                {
                    float pf[V];
                    unpack<T>(prev, pf);
                    #pragma unroll
                    for (int k = 0; k < W - 1; ++k) xx[k] = pf[V - (W - 1) + k];
                }
                unpack<T>(raw[j], xx + (W - 1));
                float o[V];
                #pragma unroll
                for (int i = 0; i < V; ++i) {
                    float acc = bv;
                    #pragma unroll
                    for (int k = 0; k < W; ++k) acc = fmaf(wv[k], xx[i + k], acc);
                    o[i] = !kSilu ? acc : (kTanh ? silu_half_arg(acc) : silu_f(acc));
                }
                store_row_vec<T, kFull>(outr, e, L, o);
            }
            carry = raw[kVecs - 1];
        }
    }
}

// ---- 16-bit I/O, rows of a multiple of 16 elements, 32-byte aligned: 32 bytes per lane --------
// A lane owns slots of 16 consecutive elements (two 16-byte vectors A, B moved by one 256-bit
// load / store; a warp instruction covers 1 KB of the row).  The arithmetic runs on fp32 pairs
// (A[i], B[i]) (FFMA2): B's left halo is A's tail, already in the lane, so only A's halo (the
// previous lane's B tail, 2 shuffles per 16 elements) crosses lanes.
#ifndef CC1D_FWD_WIDE
#define CC1D_FWD_WIDE 1
#endif
#ifndef CC1D_FWD_WIDE_THREADS
#define CC1D_FWD_WIDE_THREADS 256
#endif
#ifndef CC1D_FWD_WIDE_MINBLK
#define CC1D_FWD_WIDE_MINBLK 4       // 64 registers, 32 warps per SM
#endif
__device__ __forceinline__ void fwd_ld32(uint4 &a, uint4 &b, const void *p) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p));
}
__device__ __forceinline__ void fwd_st32(void *p, const uint4 &a, const uint4 &b) {
    asm volatile("st.global.cs.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :: "l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w) : "memory");
}

// kWhole: every slot of the row is complete; otherwise seqlen is only a multiple of 16 and a lane's 16
// elements are either all inside the row or all past its end (nothing loaded, nothing stored).
template <typename T, int W, bool kSilu, int kSlots, bool kWhole>
__global__ void __launch_bounds__(CC1D_FWD_WIDE_THREADS, CC1D_FWD_WIDE_MINBLK) fwd_cf_wide_kernel(const FwdCfArgs a) {
    pdl_wait();
    static_assert(sizeof(T) == 2, "16-bit I/O only");
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
    constexpr uint32_t kSlotElems = 32 * 16, kGroupElems = kSlots * kSlotElems;
    const int lane = threadIdx.x & 31;
    const int src_prev = (lane + 31) & 31;
    const uint32_t warps_per_cta = blockDim.x >> 5;
    const uint32_t nwarps = gridDim.x * warps_per_cta;

    for (uint32_t unit = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); unit < a.n_units; unit += nwarps) {
        const uint32_t row = unit / a.upr;
        const uint32_t seg = unit - row * a.upr;
        const uint32_t b = row / a.dim;
        const uint32_t c = row - b * a.dim;
        const T *__restrict__ xr = reinterpret_cast<const T *>(a.x) + b * a.x_bs + c * a.x_cs;
        T *__restrict__ outr = reinterpret_cast<T *>(a.out) + b * a.o_bs + c * a.o_cs;
        const uint32_t g0 = seg * a.gpu;
        const uint32_t g1 = g0 + a.gpu < a.gpr ? g0 + a.gpu : a.gpr;

        const uint32_t L = a.seqlen;
        uint4 xa[kSlots], xb[kSlots];
        #pragma unroll
        for (int j = 0; j < kSlots; ++j) {
            const uint32_t e = g0 * kGroupElems + j * kSlotElems + lane * 16;
            xa[j] = xb[j] = make_uint4(0, 0, 0, 0);
            if (kWhole || e < L) fwd_ld32(xa[j], xb[j], xr + e);
        }
        // lane 31: the 4 elements of x before the group (zeros at the row start)
        uint32_t cz = 0, cw = 0;
        if (lane == 31 && g0 > 0) {
            const uint2 t = *reinterpret_cast<const uint2 *>(xr + g0 * kGroupElems - 4);
            cz = t.x; cw = t.y;
        }
        const float pre = kTanh ? 0.5f : 1.f;     // the tanh form of SiLU works on y/2
        float2 wv[W];
        #pragma unroll
        for (int k = 0; k < W; ++k) wv[k] = splat2(pre * load_w(a.weight, c * a.w_cs + k * a.w_ws, a.wtype));
        const float2 bv = splat2(a.bias != nullptr ? pre * load_w(a.bias, c, a.wtype) : 0.f);

        for (uint32_t g = g0; g < g1; ++g) {
            #pragma unroll
            for (int j = 0; j < kSlots; ++j) {
                // left halo of A: the previous lane's B tail; lane 0 gets what lane 31 holds of the slot before
                const uint32_t oz = j > 0 ? xb[j > 0 ? j - 1 : 0].z : cz, ow = j > 0 ? xb[j > 0 ? j - 1 : 0].w : cw;
                uint32_t pz = 0;
                if (W >= 4) pz = __shfl_sync(kFullMask, lane == 31 ? oz : xb[j].z, src_prev);
                const uint32_t pw = __shfl_sync(kFullMask, lane == 31 ? ow : xb[j].w, src_prev);
                float2 xx[W - 1 + 8];
                {
                    const float2 pa = unpack_pair<T>(pz), pb = unpack_pair<T>(pw);
                    const float p[4] = {pa.x, pa.y, pb.x, pb.y};   // elements 4..7 of the vector before A
                    float af[8], bf[8];
                    unpack<T>(xa[j], af); unpack<T>(xb[j], bf);
                    #pragma unroll
                    for (int k = 0; k < W - 1; ++k) xx[k] = make_float2(p[4 - (W - 1) + k], af[8 - (W - 1) + k]);
                    #pragma unroll
                    for (int i = 0; i < 8; ++i) xx[W - 1 + i] = make_float2(af[i], bf[i]);
                }
                float o0[8], o1[8];
                #pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float2 y = bv;
                    #pragma unroll
                    for (int k = 0; k < W; ++k) y = fma2(wv[k], xx[i + k], y);
                    if (kSilu) {
                        if (kTanh) y = fma2(y, make_float2(tanh_approx(y.x), tanh_approx(y.y)), y);   // silu(2h) = h + h tanh(h)
                        else y = make_float2(silu_f(y.x), silu_f(y.y));
                    }
                    o0[i] = y.x; o1[i] = y.y;
                }
                const uint32_t e = g * kGroupElems + j * kSlotElems + lane * 16;
                if (kWhole || e < L) fwd_st32(outr + e, pack<T>(o0), pack<T>(o1));
            }
            if (g + 1 < g1) {
                // lane 31 keeps the tail of the group for lane 0 of the next one, then the next group's vectors
                cz = xb[kSlots - 1].z; cw = xb[kSlots - 1].w;
                #pragma unroll
                for (int j = 0; j < kSlots; ++j) {
                    const uint32_t e = (g + 1) * kGroupElems + j * kSlotElems + lane * 16;
                    xa[j] = xb[j] = make_uint4(0, 0, 0, 0);
                    if (kWhole || e < L) fwd_ld32(xa[j], xb[j], xr + e);
                }
            }
        }
    }
}

// Any alignment / row stride: one output element per thread, lanes along seqlen.
template <typename T, int W, bool kSilu>
__global__ void __launch_bounds__(256) fwd_cf_scalar_kernel(const FwdCfArgs a) {
    pdl_wait();
    // here: vpr = 256-element tiles per row, n_units = rows * vpr
    for (uint32_t tile = blockIdx.x; tile < a.n_units; tile += gridDim.x) {
        const uint32_t row = tile / a.vpr;
        const uint32_t t = (tile - row * a.vpr) * 256 + threadIdx.x;
        if (t >= a.seqlen) continue;
        const uint32_t b = row / a.dim;
        const uint32_t c = row - b * a.dim;
        const T *__restrict__ xr = reinterpret_cast<const T *>(a.x) + b * a.x_bs + c * a.x_cs;
        T *__restrict__ outr = reinterpret_cast<T *>(a.out) + b * a.o_bs + c * a.o_cs;
        float acc = a.bias != nullptr ? load_w(a.bias, c, a.wtype) : 0.f;
        #pragma unroll
        for (int k = 0; k < W; ++k) {
            const int64_t p = (int64_t)t - (W - 1 - k);
            if (p >= 0) acc = fmaf(load_w(a.weight, c * a.w_cs + k * a.w_ws, a.wtype), Elem<T>::to_f(xr[p]), acc);
        }
        outr[t] = Elem<T>::from_f(kSilu ? silu_f(acc) : acc);
    }
}

// Groups of one row handled by one warp: as many as possible (per-unit costs amortise, fewer
// partial rows in the backward) while leaving enough units to balance ~148 SMs x 48 warps.
uint64_t groups_per_unit(uint64_t rows, uint64_t groups_per_row) {
    const uint64_t units_wanted = 148ull * 48 * 4;
    uint64_t gpu = groups_per_row;
    while (gpu > 1 && rows * ((groups_per_row + gpu - 1) / gpu) < units_wanted) gpu = (gpu + 1) / 2;
    return gpu > 0 ? gpu : 1;
}

int launch_fwd_channel_first(const cc1d_fwd_params &p, cudaStream_t stream) {
    const int V = vec_elems(p.itype);
    const uint64_t rows = (uint64_t)p.batch * (uint64_t)p.dim;
    if (rows == 0 || p.seqlen == 0) return CC1D_OK;
    if (p.seqlen >= (1ll << 31) - 4096 || p.dim >= (1ll << 31)) return CC1D_ERR_TOO_LARGE;

    FwdCfArgs a;
    a.x = p.x; a.out = p.out; a.weight = p.weight; a.bias = p.bias;
    a.x_bs = p.batch > 1 ? p.x_batch_stride : 0; a.x_cs = p.dim > 1 ? p.x_c_stride : 0;
    a.o_bs = p.batch > 1 ? p.out_batch_stride : 0; a.o_cs = p.dim > 1 ? p.out_c_stride : 0;
    a.w_cs = p.weight_c_stride; a.w_ws = p.weight_width_stride;
    a.dim = (uint32_t)p.dim; a.seqlen = (uint32_t)p.seqlen; a.wtype = p.wtype;

    const bool vec_ok = is_aligned16(p.x) && is_aligned16(p.out) && a.x_bs % V == 0 && a.x_cs % V == 0 &&
                        a.o_bs % V == 0 && a.o_cs % V == 0;
    if (vec_ok) {
        constexpr int kVecs = kCfVecs;
        const uint64_t vpr = ((uint64_t)p.seqlen + V - 1) / V;
        const uint64_t gpr = (vpr + 32 * kVecs - 1) / (32 * kVecs);
        const uint64_t gpu = groups_per_unit(rows, gpr);
        const uint64_t upr = (gpr + gpu - 1) / gpu;
        const uint64_t n_units = rows * upr;
        if (n_units >= (1ull << 31)) return CC1D_ERR_TOO_LARGE;   // unit + grid stride must not wrap 32 bits
        a.vpr = (uint32_t)vpr; a.gpr = (uint32_t)gpr; a.gpu = (uint32_t)gpu; a.upr = (uint32_t)upr;
        a.n_units = (uint32_t)n_units;
        const uint64_t ctas = (n_units + 7) / 8;
        const bool full = p.seqlen % V == 0 && vpr % (32 * kVecs) == 0;
        const bool wide = CC1D_FWD_WIDE && kCfVecs % 2 == 0 && p.itype != CC1D_F32 && p.seqlen % 16 == 0 &&
                          ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.out)) & 31u) == 0 &&
                          (a.x_bs | a.x_cs | a.o_bs | a.o_cs) % 16 == 0;
        if (wide) {
            const uint64_t wctas = (n_units + CC1D_FWD_WIDE_THREADS / 32 - 1) / (CC1D_FWD_WIDE_THREADS / 32);
            if (p.itype == CC1D_BF16) {
                using T = __nv_bfloat16;
                CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu, CC1D_DISPATCH_BOOL(full, kWhole, {
                    launch_k(fwd_cf_wide_kernel<T, W, kSilu, kCfVecs / 2, kWhole>, dim3((unsigned)wctas), dim3(CC1D_FWD_WIDE_THREADS), 0, stream, a);
                });););
            } else {
                using T = __half;
                CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu, CC1D_DISPATCH_BOOL(full, kWhole, {
                    launch_k(fwd_cf_wide_kernel<T, W, kSilu, kCfVecs / 2, kWhole>, dim3((unsigned)wctas), dim3(CC1D_FWD_WIDE_THREADS), 0, stream, a);
                });););
            }
        } else
        CC1D_DISPATCH_ITYPE(p.itype, CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu,
            CC1D_DISPATCH_BOOL(full, kFull, {
                auto kernel = fwd_cf_vec_kernel<T, W, kSilu, kFull, kVecs>;
                // memory-bound: fresh CTAs keep more loads in flight than a grid-stride loop does
                launch_k(kernel, dim3(persistent_grid(kernel, 256, ctas, CC1D_CF_FWD_PERSISTENT != 0)), dim3(256), 0, stream, a);
            }););););
    } else {
        const uint64_t tpr = ((uint64_t)p.seqlen + 255) / 256;
        const uint64_t n_tiles = rows * tpr;
        if (n_tiles >= (1ull << 31)) return CC1D_ERR_TOO_LARGE;   // tile + grid stride must not wrap 32 bits
        a.vpr = (uint32_t)tpr; a.gpr = a.gpu = a.upr = 0; a.n_units = (uint32_t)n_tiles;
        CC1D_DISPATCH_ITYPE(p.itype, CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu, {
            auto kernel = fwd_cf_scalar_kernel<T, W, kSilu>;
            launch_k(kernel, dim3(persistent_grid(kernel, 256, n_tiles)), dim3(256), 0, stream, a);
        });););
    }
    return check_launch();
}

// ======================================================================================
// channel-last
// ======================================================================================
struct FwdClArgs {
    const void *x;
    void *out;
    const void *weight;
    const void *bias;
    const int32_t *seq_idx;
    const void *init;
    void *fin;
    int64_t x_bs, x_ls, o_bs, o_ls, w_cs, w_ws, i_bs, i_ls, f_bs, f_ls;
    int64_t dim, seqlen;
    int wtype;
    int tpt;            // tokens per thread
    uint32_t ncols;     // 16-byte channel vectors per token
    uint32_t ncolblk;   // CTAs along channels (32 vectors each)
    uint32_t ngroups;   // CTAs along seqlen per batch entry (kRows chunks each)
};

#ifndef CC1D_FWD_CL_TMA
#define CC1D_FWD_CL_TMA 1
#endif
#ifndef CC1D_FWD_TMA_MINBLK
#define CC1D_FWD_TMA_MINBLK 4        // fp32 I/O: 4 CTAs (16 warps) per SM
#endif
#ifndef CC1D_FWD_TMA_MINBLK_16BIT
#define CC1D_FWD_TMA_MINBLK_16BIT 5  // 16-bit I/O: 94 registers, 5 CTAs (20 warps) per SM
#endif
constexpr int kClRows = 8;    // token chunks per CTA (threadIdx.y)
constexpr int kClUnroll = 4;  // tokens per block: loads of one block are in flight while the previous computes

// One token of the sliding window: out = act(bias + sum_k w[k] * window[k]), then shift.
// Arithmetic on fp32 pairs of adjacent channels (FFMA2: two multiply-adds per issue slot; the
// pairs are what unpacking a 16-bit x 2 word yields, so no register moves are needed to form them).
template <typename T, int W, int C, bool kSilu, bool kSeqIdx, bool kTanh>
__device__ __forceinline__ void fwd_cl_token_impl(const Raw<T, C> &raw, int sid, float2 (&win)[W - 1][C / 2], int (&sw)[W - 1],
                                                  const float2 (&wv)[W][C / 2], const float2 (&bv)[C / 2], char *optr, bool store) {
    constexpr int P = C / 2;
    float2 cur[P], o[P];
    unpack_pairs<T>(raw, cur);
    #pragma unroll
    for (int c = 0; c < P; ++c) {
        float2 acc = bv[c];
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) {
            if (!kSeqIdx || sw[k] == sid) acc = fma2(wv[k][c], win[k][c], acc);
        }
        acc = fma2(wv[W - 1][c], cur[c], acc);
        if (kSilu) {
            if (kTanh) acc = fma2(acc, make_float2(tanh_approx(acc.x), tanh_approx(acc.y)), acc);   // silu(2h) = h + h tanh(h)
            else acc = make_float2(silu_f(acc.x), silu_f(acc.y));
        }
        // a padded token (seq_idx < 0) outputs exactly zero: no bias, no activation
        o[c] = (kSeqIdx && sid < 0) ? make_float2(0.f, 0.f) : acc;
    }
    if (store) st_stream_raw(optr, PackPairs<T, C>::run(o));
    #pragma unroll
    for (int k = 0; k < W - 2; ++k) {
        #pragma unroll
        for (int c = 0; c < P; ++c) win[k][c] = win[k + 1][c];
        if (kSeqIdx) sw[k] = sw[k + 1];
    }
    #pragma unroll
    for (int c = 0; c < P; ++c) win[W - 2][c] = cur[c];
    // unmasked code only ever runs when every id in the window already equals sid (or there are no ids)
    if (kSeqIdx) sw[W - 2] = sid;
}
template <typename T, int W, int C, bool kSilu, bool kSeqIdx, bool kTanh>
__device__ __forceinline__ void fwd_cl_token(const Raw<T, C> &raw, int sid, float2 (&win)[W - 1][C / 2], int (&sw)[W - 1],
                                             const float2 (&wv)[W][C / 2], const float2 (&bv)[C / 2], char *optr, bool store = true) {
    if (kSeqIdx) {
        bool same = sid >= 0;
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) same = same && sw[k] == sid;
        if (same) {
            fwd_cl_token_impl<T, W, C, kSilu, false, kTanh>(raw, sid, win, sw, wv, bv, optr, store);
            return;
        }
    }
    fwd_cl_token_impl<T, W, C, kSilu, kSeqIdx, kTanh>(raw, sid, win, sw, wv, bv, optr, store);
}

template <typename T, int W, bool kSilu, bool kSeqIdx>
__global__ void __launch_bounds__(32 * kClRows, 2) fwd_cl_kernel(const FwdClArgs a) {
    pdl_wait();
    constexpr int C = Elem<T>::kVec;  // channels per thread (one 16-byte vector)
    constexpr int U = kClUnroll;
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
    using R = Raw<T, C>;

    const uint32_t cb = blockIdx.x % a.ncolblk;
    const uint32_t rest = blockIdx.x / a.ncolblk;
    const uint32_t grp = rest % a.ngroups;
    const uint32_t b = rest / a.ngroups;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const uint32_t col = cb * 32 + tx;
    const int L = (int)a.seqlen;
    const int t0 = (int)((grp * kClRows + ty) * (uint32_t)a.tpt);
    if (col >= a.ncols || t0 >= L) return;
    const int t1 = t0 + a.tpt < L ? t0 + a.tpt : L;

    const int64_t xs = a.x_ls * (int64_t)sizeof(T), os = a.o_ls * (int64_t)sizeof(T);   // token strides in bytes
    const char *xptr = reinterpret_cast<const char *>(a.x) + (b * a.x_bs + (int64_t)col * C) * (int64_t)sizeof(T) + t0 * xs;
    char *optr = reinterpret_cast<char *>(a.out) + (b * a.o_bs + (int64_t)col * C) * (int64_t)sizeof(T) + t0 * os;
    const int32_t *__restrict__ sp = kSeqIdx ? a.seq_idx + (int64_t)b * L + t0 : nullptr;

    // first block of tokens and the window in front of it: all requested before the taps
    const int n = t1 - t0, nfull = n / U;
    R raw[U];
    int sid[U];
    #pragma unroll
    for (int u = 0; u < U; ++u) {
        zero_raw(raw[u]);
        sid[u] = 0;
        if (u < n) {
            ld_stream_raw(raw[u], xptr + u * xs);
            if (kSeqIdx) sid[u] = sp[u];
        }
    }
    // window = the width-1 tokens before t0 (x, or initial_states, or zero)
    float2 win[W - 1][C / 2];
    int sw[W - 1];
    #pragma unroll
    for (int k = 0; k < W - 1; ++k) {
        const int p = t0 - (W - 1) + k;
        R r;
        zero_raw(r);
        sw[k] = -1;
        if (p >= 0) {
            ld_cached_raw(r, xptr - (W - 1 - k) * xs);
            if (kSeqIdx) sw[k] = sp[k - (W - 1)];
        } else if (a.init != nullptr) {
            ld_cached_raw(r, reinterpret_cast<const T *>(a.init) + b * a.i_bs + (p + (W - 1)) * a.i_ls + (int64_t)col * C);
        }
        unpack_pairs<T>(r, win[k]);
    }
    float2 wv[W][C / 2], bv[C / 2];
    load_taps_pairs<W, C>(wv, bv, a.weight, a.w_cs, a.w_ws, a.bias, a.wtype, (int64_t)col * C, kTanh ? 0.5f : 1.f);

    // full blocks: the next block's loads are issued before the current block is computed
    for (int blk = 0; blk < nfull; ++blk) {
        R nxt[U];
        int nsid[U];
        const int left = n - (blk + 1) * U;   // tokens after this block
        #pragma unroll
        for (int u = 0; u < U; ++u) {
            zero_raw(nxt[u]);
            nsid[u] = 0;
            if (u < left) {
                ld_stream_raw(nxt[u], xptr + (U + u) * xs);
                if (kSeqIdx) nsid[u] = sp[U + u];
            }
        }
        #pragma unroll
        for (int u = 0; u < U; ++u) fwd_cl_token<T, W, C, kSilu, kSeqIdx, kTanh>(raw[u], sid[u], win, sw, wv, bv, optr + u * os);
        xptr += U * xs;
        optr += U * os;
        if (kSeqIdx) sp += U;
        #pragma unroll
        for (int u = 0; u < U; ++u) { raw[u] = nxt[u]; sid[u] = nsid[u]; }
    }
    // ragged tail (already loaded)
    #pragma unroll
    for (int u = 0; u < U; ++u) {
        if (u < n - nfull * U) fwd_cl_token<T, W, C, kSilu, kSeqIdx, kTanh>(raw[u], sid[u], win, sw, wv, bv, optr + u * os);
    }

    // the thread that consumed the last token holds the last width-1 entries of [initial | x]
    if (a.fin != nullptr && t1 == L) {
        T *fp = reinterpret_cast<T *>(a.fin) + b * a.f_bs + (int64_t)col * C;
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) st_plain_raw(fp + k * a.f_ls, PackPairs<T, C>::run(win[k]));
    }
}

// ---- TMA variant ----------------------------------------------------------------------------
// Same sliding-window arithmetic, but x reaches the warp through the TMA unit: each warp is an
// independent pipeline over its own ring of kTmaStages boxes ([kTmaRows tokens x 512 bytes]) in
// shared memory, one mbarrier per box.  Lane 0 requests boxes kTmaStages ahead; all lanes wait
// on the box's barrier, read their 16 bytes per token with ld.shared and store results
// straight to global memory.  Rows past seqlen and channels past dim are zero-filled by the
// TMA unit, so the loop has no load predicates.  Warps never synchronise with each other.
#ifndef CC1D_TMA_WARPS
#define CC1D_TMA_WARPS 4
#endif
#ifndef CC1D_TMA_STAGES
#define CC1D_TMA_STAGES 3
#endif
constexpr int kTmaWarps = CC1D_TMA_WARPS;
constexpr int kTmaStages = CC1D_TMA_STAGES;

// A thread owns kFwdTmaC = 4 adjacent channels (8 bytes of a 16-bit tensor, 16 of an fp32 one): with 8
// channels of a 16-bit tensor per thread the kernel needed 128 registers and ran 16 warps per SM at 0.94
// of the copy rate on (1,5376,32768) bf16; with 4 it needs 94, runs 20 and reaches 0.99 (bit-identical).
constexpr int kFwdTmaC = 4;
template <typename T> struct FwdTma {
    static constexpr int kRowBytes = 32 * kFwdTmaC * (int)sizeof(T);     // one token of a warp's strip
    static constexpr int kStageBytes = kTmaRows * kRowBytes;
    static constexpr size_t kSmem = (size_t)kTmaWarps * kTmaStages * kStageBytes + (size_t)kTmaWarps * kTmaStages * 8;
    static constexpr int kMinBlocks = sizeof(T) == 4 ? CC1D_FWD_TMA_MINBLK : CC1D_FWD_TMA_MINBLK_16BIT;
};
template <typename R> __device__ __forceinline__ R fwd_lds(uint32_t addr);
template <> __device__ __forceinline__ uint4 fwd_lds<uint4>(uint32_t addr) { return lds128(addr); }
template <> __device__ __forceinline__ uint2 fwd_lds<uint2>(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

template <typename T, int W, bool kSilu, bool kSeqIdx>
__global__ void __launch_bounds__(32 * kTmaWarps, FwdTma<T>::kMinBlocks)
fwd_cl_tma_kernel(const FwdClArgs a, const __grid_constant__ CUtensorMap xmap) {
    pdl_wait();
    constexpr int C = kFwdTmaC;
    constexpr bool kTanh = kSilu && UseTanhSilu<T>::value;
    constexpr int kTmaRowBytes = FwdTma<T>::kRowBytes, kTmaStageBytes = FwdTma<T>::kStageBytes;   // of this I/O type
    using R = Raw<T, C>;
    extern __shared__ __align__(1024) unsigned char smem[];

    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const uint32_t cb = blockIdx.x % a.ncolblk;
    const uint32_t rest = blockIdx.x / a.ncolblk;
    const uint32_t grp = rest % a.ngroups;
    const uint32_t b = rest / a.ngroups;
    const uint32_t col = cb * 32 + lane;
    const bool lane_ok = col < a.ncols;            // lanes past dim compute on zeros and never store
    const int L = (int)a.seqlen;
    const int t0 = (int)((grp * kTmaWarps + wid) * (uint32_t)a.tpt);
    if (t0 >= L) return;                           // whole warp
    const int t1 = t0 + a.tpt < L ? t0 + a.tpt : L;
    const int n = t1 - t0, nst = (n + kTmaRows - 1) / kTmaRows;

    const uint32_t ring = smem_u32(smem) + wid * (kTmaStages * kTmaStageBytes);
    const uint32_t bars = smem_u32(smem) + kTmaWarps * kTmaStages * kTmaStageBytes + wid * (kTmaStages * 8);
    if (lane == 0) {
        tma_prefetch_desc(&xmap);
        #pragma unroll
        for (int s = 0; s < kTmaStages; ++s) mbar_init(bars + 8 * s, 1);
        fence_mbar_init();
        #pragma unroll
        for (int s = 0; s < kTmaStages; ++s) {
            if (s < nst) {
                mbar_expect_tx(bars + 8 * s, kTmaStageBytes);
                tma_load_3d(ring + s * kTmaStageBytes, &xmap, (int)(cb * 32 * C), t0 + s * kTmaRows, (int)b, bars + 8 * s);
            }
        }
    }
    __syncwarp();

    const int64_t xs = a.x_ls * (int64_t)sizeof(T), os = a.o_ls * (int64_t)sizeof(T);
    const char *xptr = reinterpret_cast<const char *>(a.x) + (b * a.x_bs + (int64_t)col * C) * (int64_t)sizeof(T) + t0 * xs;
    char *optr = reinterpret_cast<char *>(a.out) + (b * a.o_bs + (int64_t)col * C) * (int64_t)sizeof(T) + t0 * os;
    const int32_t *__restrict__ sp = kSeqIdx ? a.seq_idx + (int64_t)b * L + t0 : nullptr;

    // window = the width-1 tokens before t0 (x, or initial_states, or zero)
    float2 win[W - 1][C / 2];
    int sw[W - 1];
    #pragma unroll
    for (int k = 0; k < W - 1; ++k) {
        const int p = t0 - (W - 1) + k;
        R r;
        zero_raw(r);
        sw[k] = -1;
        if (p >= 0) {
            if (lane_ok) ld_cached_raw(r, xptr - (W - 1 - k) * xs);
            if (kSeqIdx) sw[k] = sp[k - (W - 1)];
        } else if (a.init != nullptr && lane_ok) {
            ld_cached_raw(r, reinterpret_cast<const T *>(a.init) + b * a.i_bs + (p + (W - 1)) * a.i_ls + (int64_t)col * C);
        }
        unpack_pairs<T>(r, win[k]);
    }
    float2 wv[W][C / 2], bv[C / 2];
    if (lane_ok) {
        load_taps_pairs<W, C>(wv, bv, a.weight, a.w_cs, a.w_ws, a.bias, a.wtype, (int64_t)col * C, kTanh ? 0.5f : 1.f);
    } else {
        #pragma unroll
        for (int c = 0; c < C / 2; ++c) {
            bv[c] = make_float2(0.f, 0.f);
            #pragma unroll
            for (int k = 0; k < W; ++k) wv[k][c] = make_float2(0.f, 0.f);
        }
    }

    // sequence ids of a box are fetched one box ahead, so that their latency hides behind a box;
    // one id per lane: lane l holds the id of row l % kTmaRows (-2 past the chunk: matches nothing)
    const int myrow = lane & (kTmaRows - 1);
    int next_id = (kSeqIdx && myrow < n) ? sp[myrow] : -2;
    for (int st = 0; st < nst; ++st) {
        const int s = st % kTmaStages;
        const int rows = n - st * kTmaRows;            // >= kTmaRows except in the last box
        const int my_id = next_id;
        next_id = (kSeqIdx && kTmaRows + myrow < rows) ? sp[kTmaRows + myrow] : -2;
        if (!__all_sync(kFullMask, mbar_wait(bars + 8 * s, (uint32_t)(st / kTmaStages) & 1u))) {   // the warp decides together
            g_tma_wait_expired = 1;                    // never expected; leave without touching more memory
            return;
        }
        const uint32_t src = ring + s * kTmaStageBytes + lane * (C * (int)sizeof(T));
        // one test per box instead of one per token: a box whose tokens and window all carry the
        // same non-negative sequence id needs no masking at all (warp-uniform branch)
        bool plain = rows >= kTmaRows;
        if (kSeqIdx) {
            const int first = __shfl_sync(kFullMask, my_id, 0);
            bool same = my_id == first && first >= 0;
            #pragma unroll
            for (int k = 0; k < W - 1; ++k) same = same && sw[k] == first;
            plain = __all_sync(kFullMask, same) && plain;
        }
        int sid[kTmaRows];       // per-row ids: only the masked paths look at them
        if (!plain) {
            #pragma unroll
            for (int r = 0; r < kTmaRows; ++r) sid[r] = kSeqIdx ? __shfl_sync(kFullMask, my_id, r) : 0;
        }
        if (plain) {
            #pragma unroll
            for (int r = 0; r < kTmaRows; ++r) {
                const R raw = fwd_lds<R>(src + r * kTmaRowBytes);
                fwd_cl_token_impl<T, W, C, kSilu, false, kTanh>(raw, 0, win, sw, wv, bv, optr + r * os, lane_ok);
            }
        } else if (rows >= kTmaRows) {
            #pragma unroll
            for (int r = 0; r < kTmaRows; ++r) {
                const R raw = fwd_lds<R>(src + r * kTmaRowBytes);
                fwd_cl_token_impl<T, W, C, kSilu, kSeqIdx, kTanh>(raw, sid[r], win, sw, wv, bv, optr + r * os, lane_ok);
            }
        } else {
            #pragma unroll
            for (int r = 0; r < kTmaRows; ++r) {
                if (r < rows) {
                    const R raw = fwd_lds<R>(src + r * kTmaRowBytes);
                    fwd_cl_token<T, W, C, kSilu, kSeqIdx, kTanh>(raw, sid[r], win, sw, wv, bv, optr + r * os, lane_ok);
                }
            }
        }
        optr += kTmaRows * os;
        if (kSeqIdx) sp += kTmaRows;
        __syncwarp();                                   // every lane has consumed the box
        if (lane == 0 && st + kTmaStages < nst) {       // refill it
            fence_proxy_async_smem();
            mbar_expect_tx(bars + 8 * s, kTmaStageBytes);
            tma_load_3d(ring + s * kTmaStageBytes, &xmap, (int)(cb * 32 * C), t0 + (st + kTmaStages) * kTmaRows, (int)b,
                        bars + 8 * s);
        }
    }

    // the thread that consumed the last token holds the last width-1 entries of [initial | x]
    if (a.fin != nullptr && t1 == L && lane_ok) {
        T *fp = reinterpret_cast<T *>(a.fin) + b * a.f_bs + (int64_t)col * C;
        #pragma unroll
        for (int k = 0; k < W - 1; ++k) st_plain_raw(fp + k * a.f_ls, PackPairs<T, C>::run(win[k]));
    }
}

// Tokens per thread: long enough to amortise the (width-1)-token halo re-read, short enough
// to fill the machine (~2 CTAs of 256 threads per SM and more).
int pick_tokens_per_thread(int64_t batch, int64_t ncols, int64_t seqlen, int sms, int max_tpt) {
    const double threads_wanted = (double)sms * 2048.0;
    const double cols_total = (double)batch * (double)ncols;
    int tpt = max_tpt;
    while (tpt > 8 && cols_total * (double)((seqlen + tpt - 1) / tpt) < threads_wanted) tpt >>= 1;
    return tpt;
}

// Chunk length (tokens a warp walks) for the TMA kernels on a problem of several waves.  The grid runs in
// waves of `resident_ctas`; a chunk costs its tokens plus about `overhead` tokens of prologue, halo and
// epilogue; the candidate with the smallest waves x (tokens + overhead) wins, the first one on a tie.
int pick_chunk_tokens(int64_t batch, int64_t ncolblk, int64_t seqlen, int warps_per_cta, int64_t resident_ctas,
                      const int *candidates, int n, int overhead) {
    int best = candidates[0];
    double best_cost = 0.0;
    for (int i = 0; i < n; ++i) {
        const int tpt = candidates[i];
        const int64_t chunks = (seqlen + tpt - 1) / tpt;
        const int64_t groups = (chunks + warps_per_cta - 1) / warps_per_cta;
        const double ctas = (double)ncolblk * (double)groups * (double)batch;
        const double waves = ceil(ctas / (double)resident_ctas);
        const double cost = waves * (double)(tpt + overhead);
        if (i == 0 || cost < best_cost) { best = tpt; best_cost = cost; }
    }
    return best;
}

int launch_fwd_channel_last(const cc1d_fwd_params &p, cudaStream_t stream) {
    if (p.batch == 0 || p.dim == 0 || p.seqlen == 0) return CC1D_OK;
    // token positions are 32-bit integers in the kernels (chunk starts plus a halo must not wrap)
    if (p.seqlen >= (1ll << 31) - 4096 || p.dim >= (1ll << 31)) return CC1D_ERR_TOO_LARGE;
    const int C = vec_elems(p.itype);
    if (!is_aligned16(p.x) || !is_aligned16(p.out)) return CC1D_ERR_ALIGN;
    if (p.initial_states && (!is_aligned16(p.initial_states) || p.initial_states_batch_stride % C ||
                             p.initial_states_l_stride % C)) return CC1D_ERR_ALIGN;
    if (p.final_states && (!is_aligned16(p.final_states) || p.final_states_batch_stride % C ||
                           p.final_states_l_stride % C)) return CC1D_ERR_ALIGN;
    const int sms = num_sms();
    FwdClArgs a;
    a.x = p.x; a.out = p.out; a.weight = p.weight; a.bias = p.bias; a.seq_idx = p.seq_idx;
    a.init = p.initial_states; a.fin = p.final_states;
    a.x_bs = p.x_batch_stride; a.x_ls = p.x_l_stride; a.o_bs = p.out_batch_stride; a.o_ls = p.out_l_stride;
    a.w_cs = p.weight_c_stride; a.w_ws = p.weight_width_stride;
    a.i_bs = p.initial_states_batch_stride; a.i_ls = p.initial_states_l_stride;
    a.f_bs = p.final_states_batch_stride; a.f_ls = p.final_states_l_stride;
    a.dim = p.dim; a.seqlen = p.seqlen; a.wtype = p.wtype;
    const int64_t ncols = p.dim / C;
    a.tpt = pick_tokens_per_thread(p.batch, ncols, p.seqlen, sms, 64);
#ifndef CC1D_TMA_TPT
#define CC1D_TMA_TPT 64
#endif
    a.ncols = (uint32_t)ncols;
    a.ncolblk = (uint32_t)((ncols + 31) / 32);
    const int64_t chunks = (p.seqlen + a.tpt - 1) / a.tpt;
    a.ngroups = (uint32_t)((chunks + kClRows - 1) / kClRows);
#if CC1D_FWD_CL_TMA
    // TMA path, 4 channels per thread for every I/O type (fp32 (8,5120,2048): 105 us against 120 us with the
    // register-prefetch kernel below, which stays for tensors the driver refuses a map for)
    CUtensorMap xmap;
    if (p.seqlen < (1ll << 31) && p.batch < (1ll << 31) &&
        make_channel_last_tensor_map(&xmap, p.itype, p.x, p.dim, p.seqlen, p.batch, p.x_l_stride, p.x_batch_stride,
                                     32 * kFwdTmaC * elem_size(p.itype))) {
        FwdClArgs t = a;
        const int64_t tcols = p.dim / kFwdTmaC;
        t.ncols = (uint32_t)tcols;
        t.ncolblk = (uint32_t)((tcols + 31) / 32);
        // each warp keeps kTmaStages boxes in flight, so fewer and longer chunks fill the machine
        if (p.itype == CC1D_F32) {
            t.tpt = pick_tokens_per_thread(p.batch, tcols, p.seqlen, sms / 2, CC1D_TMA_TPT);
            if (t.tpt == 64) {
                // several waves: pick the chunk by the waves it makes (measured with 8 channels per thread, bf16
                // (8,5120,2048): 64 tokens, 4.3 waves, 61.4 us; 48 tokens, 5.95 waves, 57.6 us)
                static const int kChunks[] = {64, 56, 48};
                t.tpt = pick_chunk_tokens(p.batch, t.ncolblk, p.seqlen, kTmaWarps, (int64_t)sms * CC1D_FWD_TMA_MINBLK, kChunks, 3, 8);
            }
        } else {
            // measured, bf16, 48 / 56 / 64 / 80 tokens: (1,5376,32768) 108.9 / 109.1 / 109.3 / 110.9 us,
            // (8,5120,2048) 54.7 / 55.5 / 55.9 / 57.2 us
            t.tpt = pick_tokens_per_thread(p.batch, tcols, p.seqlen, sms / 2, 48);
        }
        const int64_t tchunks = (p.seqlen + t.tpt - 1) / t.tpt;
        t.ngroups = (uint32_t)((tchunks + kTmaWarps - 1) / kTmaWarps);
        const uint64_t tctas = (uint64_t)t.ncolblk * t.ngroups * (uint64_t)p.batch;
        if (tctas >= (1ull << 31)) return CC1D_ERR_TOO_LARGE;
        CC1D_DISPATCH_ITYPE(p.itype, CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu,
            CC1D_DISPATCH_BOOL(p.seq_idx != nullptr, kSeqIdx, {
                auto kernel = fwd_cl_tma_kernel<T, W, kSilu, kSeqIdx>;
                allow_dynamic_smem(reinterpret_cast<const void *>(kernel), FwdTma<T>::kSmem);
                launch_k(kernel, dim3((unsigned)tctas), dim3(32 * kTmaWarps), FwdTma<T>::kSmem, stream, t, xmap);
            }););););
        return check_launch();
    }
#endif
    const uint64_t ctas = (uint64_t)a.ncolblk * a.ngroups * (uint64_t)p.batch;
    if (ctas >= (1ull << 31)) return CC1D_ERR_TOO_LARGE;
    CC1D_DISPATCH_ITYPE(p.itype, CC1D_DISPATCH_WIDTH(p.width, CC1D_DISPATCH_BOOL(p.silu != 0, kSilu,
        CC1D_DISPATCH_BOOL(p.seq_idx != nullptr, kSeqIdx, {
            launch_k(fwd_cl_kernel<T, W, kSilu, kSeqIdx>, dim3((unsigned)ctas), dim3(32 * kClRows), 0, stream, a);
        }););););
    return check_launch();
}

int fwd_wait_expired() { return read_and_clear_wait_expired(); }

}  // namespace cc1d
