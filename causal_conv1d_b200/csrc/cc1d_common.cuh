// Shared device helpers for the sm_100a causal conv1d kernels: element traits, 16-byte
// streaming loads/stores, fp32 conversion, SiLU, tap loading.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "cc1d.h"

namespace cc1d {

constexpr unsigned kFullMask = 0xffffffffu;

// ---- programmatic dependent launch ------------------------------------------------------
// First statement of every kernel: wait until the kernels before this one in the stream have
// completed (their writes visible), then let the kernel after this one be scheduled as SMs
// free up.  Both are no-ops for a launch without the programmatic-serialisation attribute.
#ifndef CC1D_PDL
#define CC1D_PDL 1
#endif
__device__ __forceinline__ void pdl_wait() {
#if CC1D_PDL
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}

// ---- element traits -----------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
    static constexpr int kVec = 4;   // elements per 16-byte vector
    static __device__ __forceinline__ float to_f(float v) { return v; }
    static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct Elem<__half> {
    static constexpr int kVec = 8;
    static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
    static constexpr int kVec = 8;
    static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// ---- 16-byte global access ------------------------------------------------------------
// Read-once input streams: non-coherent path, do not keep the line in L1.
#ifndef CC1D_STREAM_HINTS
#define CC1D_STREAM_HINTS 1
#endif
__device__ __forceinline__ uint4 ld_stream(const void *p) {
#if !CC1D_STREAM_HINTS
    return *reinterpret_cast<const uint4 *>(p);
#endif
    // volatile: a plain asm is assumed free of side effects and may be hoisted above the
    // bounds check that guards it; a load can fault, so it must stay where it is written
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// Data that another thread of the same launch may also read (halos): plain cached load.
__device__ __forceinline__ uint4 ld_cached(const void *p) {
    return *reinterpret_cast<const uint4 *>(p);
}
// Write-once output streams: evict-first.
__device__ __forceinline__ void st_stream(void *p, const uint4 &v) {
#if !CC1D_STREAM_HINTS
    *reinterpret_cast<uint4 *>(p) = v;
    return;
#endif
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- 16-byte vector <-> fp32 ------------------------------------------------------------
template <typename T> __device__ __forceinline__ void unpack(const uint4 &v, float *f);
template <> __device__ __forceinline__ void unpack<float>(const uint4 &v, float *f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}
template <> __device__ __forceinline__ void unpack<__nv_bfloat16>(const uint4 &v, float *f) {
    const uint32_t r[4] = {v.x, v.y, v.z, v.w};
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(r[i] << 16);
        f[2 * i + 1] = __uint_as_float(r[i] & 0xffff0000u);
    }
}
template <> __device__ __forceinline__ void unpack<__half>(const uint4 &v, float *f) {
    const uint32_t r[4] = {v.x, v.y, v.z, v.w};
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2 *>(&r[i]));
        f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
}

template <typename T> __device__ __forceinline__ uint4 pack(const float *f);
template <> __device__ __forceinline__ uint4 pack<float>(const float *f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]),
                      __float_as_uint(f[2]), __float_as_uint(f[3]));
}
template <> __device__ __forceinline__ uint4 pack<__nv_bfloat16>(const float *f) {
    uint32_t r[4];
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        r[i] = *reinterpret_cast<const uint32_t *>(&t);
    }
    return make_uint4(r[0], r[1], r[2], r[3]);
}
template <> __device__ __forceinline__ uint4 pack<__half>(const float *f) {
    uint32_t r[4];
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 t = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        r[i] = *reinterpret_cast<const uint32_t *>(&t);
    }
    return make_uint4(r[0], r[1], r[2], r[3]);
}

// ---- 8- or 16-byte per-lane vectors of C elements (channel-last kernels) -------------------
template <int BYTES> struct RawBytes;
template <> struct RawBytes<16> { using type = uint4; };
template <> struct RawBytes<8> { using type = uint2; };
template <typename T, int C> using Raw = typename RawBytes<sizeof(T) * C>::type;

__device__ __forceinline__ void zero_raw(uint4 &v) { v = make_uint4(0, 0, 0, 0); }
__device__ __forceinline__ void zero_raw(uint2 &v) { v = make_uint2(0, 0); }

__device__ __forceinline__ void ld_stream_raw(uint4 &v, const void *p) { v = ld_stream(p); }
__device__ __forceinline__ void ld_stream_raw(uint2 &v, const void *p) {
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
}
__device__ __forceinline__ void ld_cached_raw(uint4 &v, const void *p) { v = *reinterpret_cast<const uint4 *>(p); }
__device__ __forceinline__ void ld_cached_raw(uint2 &v, const void *p) { v = *reinterpret_cast<const uint2 *>(p); }
__device__ __forceinline__ void st_stream_raw(void *p, const uint4 &v) { st_stream(p, v); }
__device__ __forceinline__ void st_stream_raw(void *p, const uint2 &v) {
    asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" :: "l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void st_plain_raw(void *p, const uint4 &v) { *reinterpret_cast<uint4 *>(p) = v; }
__device__ __forceinline__ void st_plain_raw(void *p, const uint2 &v) { *reinterpret_cast<uint2 *>(p) = v; }

template <typename T> __device__ __forceinline__ void unpack_raw(const uint4 &v, float *f) { unpack<T>(v, f); }
template <typename T> __device__ __forceinline__ void unpack_raw(const uint2 &v, float *f);   // 4 x 16-bit
template <> __device__ __forceinline__ void unpack_raw<__nv_bfloat16>(const uint2 &v, float *f) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
}
template <> __device__ __forceinline__ void unpack_raw<__half>(const uint2 &v, float *f) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&v.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&v.y));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
template <typename T, int C> struct PackRaw;
template <typename T> struct PackRaw<T, 8> { static __device__ __forceinline__ uint4 run(const float *f) { return pack<T>(f); } };
template <> struct PackRaw<float, 4> { static __device__ __forceinline__ uint4 run(const float *f) { return pack<float>(f); } };
template <> struct PackRaw<__nv_bfloat16, 4> {
    static __device__ __forceinline__ uint2 run(const float *f) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
        return make_uint2(*reinterpret_cast<const uint32_t *>(&a), *reinterpret_cast<const uint32_t *>(&b));
    }
};
template <> struct PackRaw<__half, 4> {
    static __device__ __forceinline__ uint2 run(const float *f) {
        const __half2 a = __floats2half2_rn(f[0], f[1]), b = __floats2half2_rn(f[2], f[3]);
        return make_uint2(*reinterpret_cast<const uint32_t *>(&a), *reinterpret_cast<const uint32_t *>(&b));
    }
};

// ---- packed fp32 pairs (sm_100 FFMA2 / FMUL2 / FADD2: two fp32 operations per issue slot) --
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 splat2(float v) { return make_float2(v, v); }

// C elements of a raw vector as C/2 fp32 pairs (adjacent elements share a pair)
template <typename T> __device__ __forceinline__ float2 unpack_pair(uint32_t r);
template <> __device__ __forceinline__ float2 unpack_pair<__nv_bfloat16>(uint32_t r) {
    return make_float2(__uint_as_float(r << 16), __uint_as_float(r & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 unpack_pair<__half>(uint32_t r) {
    return __half22float2(*reinterpret_cast<const __half2 *>(&r));
}
template <typename T> __device__ __forceinline__ void unpack_pairs(const uint4 &v, float2 *f) {   // 8 x 16-bit
    f[0] = unpack_pair<T>(v.x); f[1] = unpack_pair<T>(v.y); f[2] = unpack_pair<T>(v.z); f[3] = unpack_pair<T>(v.w);
}
template <> __device__ __forceinline__ void unpack_pairs<float>(const uint4 &v, float2 *f) {       // 4 x fp32
    f[0] = make_float2(__uint_as_float(v.x), __uint_as_float(v.y));
    f[1] = make_float2(__uint_as_float(v.z), __uint_as_float(v.w));
}
template <typename T> __device__ __forceinline__ void unpack_pairs(const uint2 &v, float2 *f) {   // 4 x 16-bit
    f[0] = unpack_pair<T>(v.x); f[1] = unpack_pair<T>(v.y);
}
template <typename T> __device__ __forceinline__ uint32_t pack_pair(float2 v);
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float2 v) {
    const __nv_bfloat162 t = __floats2bfloat162_rn(v.x, v.y);
    return *reinterpret_cast<const uint32_t *>(&t);
}
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float2 v) {
    const __half2 t = __floats2half2_rn(v.x, v.y);
    return *reinterpret_cast<const uint32_t *>(&t);
}
template <typename T, int C> struct PackPairs;   // C/2 pairs -> Raw<T, C>
template <typename T> struct PackPairs<T, 8> {
    static __device__ __forceinline__ uint4 run(const float2 *f) {
        return make_uint4(pack_pair<T>(f[0]), pack_pair<T>(f[1]), pack_pair<T>(f[2]), pack_pair<T>(f[3]));
    }
};
template <typename T> struct PackPairs<T, 4> {
    static __device__ __forceinline__ uint2 run(const float2 *f) { return make_uint2(pack_pair<T>(f[0]), pack_pair<T>(f[1])); }
};
template <> struct PackPairs<float, 4> {
    static __device__ __forceinline__ uint4 run(const float2 *f) {
        return make_uint4(__float_as_uint(f[0].x), __float_as_uint(f[0].y), __float_as_uint(f[1].x), __float_as_uint(f[1].y));
    }
};

// ---- activation ---------------------------------------------------------------------------
// Two evaluations of SiLU.  "exact": sigmoid through ex2 + rcp (2 special-function ops per
// element).  "tanh": sigmoid(y) = 0.5 * tanh(y/2) + 0.5 with the hardware tanh.approx (1
// special-function op, absolute error ~2.5e-4 in sigmoid) — used for bf16 I/O only, whose
// own rounding (2^-9 relative) dominates that error; fp32 and fp16 use the exact form.
// The tanh forms take h = y/2, which callers get for free by halving weights and bias.
__device__ __forceinline__ float sigmoid_f(float y) { return __fdividef(1.f, 1.f + __expf(-y)); }
__device__ __forceinline__ float silu_f(float y) { return __fdividef(y, 1.f + __expf(-y)); }
// d silu(y) / dy
__device__ __forceinline__ float dsilu_f(float y) {
    const float s = sigmoid_f(y);
    return s * (1.f + y * (1.f - s));
}
__device__ __forceinline__ float tanh_approx(float x) {
    float r;
    asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
// silu(2h) = h + h * tanh(h)
__device__ __forceinline__ float silu_half_arg(float h) { return fmaf(h, tanh_approx(h), h); }
// Backward, tanh form without a negation: callers scale the taps of the pre-activation by -1/2
// (free), which gives hn = -y/2 and tn = tanh(hn) = -tanh(y/2); then
//     2 * silu'(y) = (1 - tn) + hn * (tn^2 - 1).
// These return dout * 2 * silu'(y): g is carried with the factor ActGrad::kGScale = 2, which
// callers take back out of the taps used for dx and out of the dweight / dbias sums (both free).
__device__ __forceinline__ float act_grad_neg_half_arg(float hn, float dout) {
    const float tn = tanh_approx(hn);
    return dout * fmaf(hn, fmaf(tn, tn, -1.f), 1.f - tn);
}
// pair form: kTanh takes hn = -y/2 and returns 2 * g (see above), otherwise y and g
template <bool kTanh> __device__ __forceinline__ float2 act_grad_pair(float2 v, float2 dout) {
    if (kTanh) {
        const float2 tn = make_float2(tanh_approx(v.x), tanh_approx(v.y));
        const float2 m = fma2(tn, tn, splat2(-1.f));
        const float2 u = fma2(tn, splat2(-1.f), splat2(1.f));
        return mul2(dout, fma2(v, m, u));
    }
    return make_float2(dout.x * dsilu_f(v.x), dout.y * dsilu_f(v.y));
}
// scale of the taps that produce the backward's pre-activation argument, and of the g it carries
template <bool kTanh> struct ActGrad {
    static constexpr float kPre = kTanh ? -0.5f : 1.f;
    static constexpr float kGScale = kTanh ? 2.f : 1.f;
};
#ifndef CC1D_TANH_SILU_FP16
#define CC1D_TANH_SILU_FP16 1
#endif
template <typename T> struct UseTanhSilu { static constexpr bool value = false; };
template <> struct UseTanhSilu<__nv_bfloat16> { static constexpr bool value = true; };
#if CC1D_TANH_SILU_FP16
template <> struct UseTanhSilu<__half> { static constexpr bool value = true; };
#endif

// ---- channel-first row access: 16-byte vectors of one (batch, channel) row -----------------
// Vector at element offset e of a row of L elements: one 16-byte load when it lies fully
// inside the row (always, when kFull), element loads for the ragged last vector, zeros beyond.
template <typename T, bool kFull>
__device__ __forceinline__ uint4 load_row_vec(const T *__restrict__ row, uint32_t e, uint32_t L) {
    constexpr int V = Elem<T>::kVec;
    if (kFull || e + V <= L) return ld_stream(row + e);
    if (e >= L) return make_uint4(0, 0, 0, 0);
    float f[V];
    #pragma unroll
    for (int i = 0; i < V; ++i) f[i] = e + i < L ? Elem<T>::to_f(row[e + i]) : 0.f;
    return pack<T>(f);
}

template <typename T, bool kFull>
__device__ __forceinline__ void store_row_vec(T *__restrict__ row, uint32_t e, uint32_t L, const float *f) {
    constexpr int V = Elem<T>::kVec;
    if (kFull || e + V <= L) {
        st_stream(row + e, pack<T>(f));
    } else {
        #pragma unroll
        for (int i = 0; i < V; ++i) {
            if (e + i < L) row[e + i] = Elem<T>::from_f(f[i]);
        }
    }
}

// The registers of the previous lane's vector that hold its trailing width-1 elements; lane 0
// receives lane 31's `old` instead (the vector that precedes lane 0's in memory).
template <int V, int W>
__device__ __forceinline__ uint4 prev_vector_tail(const uint4 &own, const uint4 &old, int lane) {
    const int src_lane = (lane + 31) & 31;
    uint4 prev = make_uint4(0, 0, 0, 0);
    if (V == 4) {
        if (W >= 4) prev.y = __shfl_sync(kFullMask, lane == 31 ? old.y : own.y, src_lane);
        if (W >= 3) prev.z = __shfl_sync(kFullMask, lane == 31 ? old.z : own.z, src_lane);
    } else {
        if (W >= 4) prev.z = __shfl_sync(kFullMask, lane == 31 ? old.z : own.z, src_lane);
    }
    prev.w = __shfl_sync(kFullMask, lane == 31 ? old.w : own.w, src_lane);
    return prev;
}

// ---- weights: dtype chosen at run time (they are a few KB, never on the critical stream) --
__device__ __forceinline__ float load_w(const void *p, int64_t idx, int wtype) {
    if (wtype == CC1D_F32) return reinterpret_cast<const float *>(p)[idx];
    if (wtype == CC1D_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[idx]);
    return __half2float(reinterpret_cast<const __half *>(p)[idx]);
}

// Taps and bias of C consecutive channels straight into registers: wv[k][c], bv[c].  When the
// weight matrix is dense row-major (taps of a channel adjacent, channels adjacent) and 16-byte
// aligned, C * W taps are fetched with 16-byte loads; any other stride pattern goes element
// by element.  `scale` is folded into both (0.5 for the tanh form of SiLU).
template <int W, int C>
__device__ __forceinline__ void load_taps(float (&wv)[W][C], float (&bv)[C], const void *weight, int64_t w_cs,
                                          int64_t w_ws, const void *bias, int wtype, int64_t c0, float scale) {
    const bool dense = w_ws == 1 && w_cs == W;
    if (dense && wtype != CC1D_F32 && (reinterpret_cast<uintptr_t>(weight) & 15) == 0 && (C * W) % 8 == 0) {
        const uint4 *p = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(weight) + c0 * W);
        float f[C * W];
        #pragma unroll
        for (int i = 0; i < C * W / 8; ++i) {
            const uint4 v = __ldg(p + i);
            if (wtype == CC1D_BF16) unpack<__nv_bfloat16>(v, f + 8 * i); else unpack<__half>(v, f + 8 * i);
        }
        #pragma unroll
        for (int c = 0; c < C; ++c) {
            #pragma unroll
            for (int k = 0; k < W; ++k) wv[k][c] = scale * f[c * W + k];
        }
    } else if (dense && wtype == CC1D_F32 && (reinterpret_cast<uintptr_t>(weight) & 15) == 0 && (C * W) % 4 == 0) {
        const uint4 *p = reinterpret_cast<const uint4 *>(reinterpret_cast<const float *>(weight) + c0 * W);
        float f[C * W];
        #pragma unroll
        for (int i = 0; i < C * W / 4; ++i) unpack<float>(__ldg(p + i), f + 4 * i);
        #pragma unroll
        for (int c = 0; c < C; ++c) {
            #pragma unroll
            for (int k = 0; k < W; ++k) wv[k][c] = scale * f[c * W + k];
        }
    } else {
        #pragma unroll
        for (int c = 0; c < C; ++c) {
            #pragma unroll
            for (int k = 0; k < W; ++k) wv[k][c] = scale * load_w(weight, (c0 + c) * w_cs + k * w_ws, wtype);
        }
    }
    #pragma unroll
    for (int c = 0; c < C; ++c) bv[c] = bias != nullptr ? scale * load_w(bias, c0 + c, wtype) : 0.f;
}

// Same, as fp32 pairs of adjacent channels: wv2[k][c/2] = (w[c][k], w[c+1][k]).
template <int W, int C>
__device__ __forceinline__ void load_taps_pairs(float2 (&wv2)[W][C / 2], float2 (&bv2)[C / 2], const void *weight,
                                                int64_t w_cs, int64_t w_ws, const void *bias, int wtype, int64_t c0,
                                                float scale) {
    float wv[W][C], bv[C];
    load_taps<W, C>(wv, bv, weight, w_cs, w_ws, bias, wtype, c0, scale);
    #pragma unroll
    for (int k = 0; k < W; ++k) {
        #pragma unroll
        for (int c = 0; c < C / 2; ++c) wv2[k][c] = make_float2(wv[k][2 * c], wv[k][2 * c + 1]);
    }
    #pragma unroll
    for (int c = 0; c < C / 2; ++c) bv2[c] = make_float2(bv[2 * c], bv[2 * c + 1]);
}

}  // namespace cc1d
