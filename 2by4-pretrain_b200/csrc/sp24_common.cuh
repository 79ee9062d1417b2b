// Shared device helpers of the sm_100a kernels: element conversion, the 2:4 selection
// and encoding rules, the metadata placement formula, MVUE arithmetic and the Philox stream.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "../../include/sparse24_b200.h"

namespace sp24 {

// ---------------------------------------------------------------------------------------------
// element types
// ---------------------------------------------------------------------------------------------
struct e4m3_t { uint8_t b; };
struct e5m2_t { uint8_t b; };

template <typename T> struct Elem;
template <> struct Elem<float> {
    static constexpr int code = SP24_F32;
    __device__ static float to_f32(float v) { return v; }
    __device__ static float from_f32(float v) { return v; }
};
template <> struct Elem<__half> {
    static constexpr int code = SP24_F16;
    __device__ static float to_f32(__half v) { return __half2float(v); }
    __device__ static __half from_f32(float v) { return __float2half_rn(v); }
    // two values rounded and packed into one register (lo in bits 0..15): one conversion instruction
    __device__ static uint32_t pack2(float lo, float hi) {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
};
template <> struct Elem<__nv_bfloat16> {
    static constexpr int code = SP24_BF16;
    __device__ static float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
    __device__ static uint32_t pack2(float lo, float hi) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
};
template <> struct Elem<e4m3_t> {
    static constexpr int code = SP24_E4M3;
    __device__ static float to_f32(e4m3_t v) {
        return __half2float(__half(__nv_cvt_fp8_to_halfraw(v.b, __NV_E4M3)));
    }
    __device__ static e4m3_t from_f32(float v) {
        return e4m3_t{(uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3)};
    }
};
template <> struct Elem<e5m2_t> {
    static constexpr int code = SP24_E5M2;
    __device__ static float to_f32(e5m2_t v) {
        return __half2float(__half(__nv_cvt_fp8_to_halfraw(v.b, __NV_E5M2)));
    }
    __device__ static e5m2_t from_f32(float v) {
        return e5m2_t{(uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E5M2)};
    }
};
template <> struct Elem<int8_t> {
    static constexpr int code = SP24_I8;
    __device__ static float to_f32(int8_t v) { return (float)v; }
    __device__ static int8_t from_f32(float v) { return (int8_t)v; }
};

// value as stored in TIn -> value stored in TOut (one rounding from the source precision)
template <typename TOut, typename TIn> __device__ __forceinline__ TOut convert(TIn v) {
    return Elem<TOut>::from_f32(Elem<TIn>::to_f32(v));
}

// ---------------------------------------------------------------------------------------------
// vector access (16-byte, or narrower when the element count demands)
// ---------------------------------------------------------------------------------------------
template <int BYTES> struct VecBytes;
template <> struct VecBytes<16> { using type = uint4; };
template <> struct VecBytes<8> { using type = uint2; };
template <> struct VecBytes<4> { using type = uint32_t; };
template <> struct VecBytes<2> { using type = uint16_t; };
template <> struct VecBytes<1> { using type = uint8_t; };

template <typename T, int N> struct alignas(sizeof(T) * N) Vec {
    T v[N];
};

template <typename T, int N> __device__ __forceinline__ Vec<T, N> load_vec(const T *p) {
    using R = typename VecBytes<sizeof(T) * N>::type;
    Vec<T, N> out;
    *reinterpret_cast<R *>(&out) = *reinterpret_cast<const R *>(p);
    return out;
}
template <typename T, int N> __device__ __forceinline__ void store_vec(T *p, const Vec<T, N> &val) {
    using R = typename VecBytes<sizeof(T) * N>::type;
    *reinterpret_cast<R *>(p) = *reinterpret_cast<const R *>(&val);
}

// ---------------------------------------------------------------------------------------------
// 2:4 selection by magnitude: six strict comparisons, ties keep the higher index.
// Returns the keep mask as bits 0..3.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t magnitude_mask4(float a0, float a1, float a2, float a3) {
    a0 = fabsf(a0); a1 = fabsf(a1); a2 = fabsf(a2); a3 = fabsf(a3);
    const bool x1 = a0 > a1, x2 = a0 > a2, x3 = a0 > a3, x4 = a1 > a2, x5 = a1 > a3, x6 = a2 > a3;
    const bool m0 = (x2 && x3) || (x1 && x2) || (x1 && x3);
    const bool m1 = (!x1 && x5) || (x4 && x5) || (!x1 && x4);
    const bool m2 = (!x2 && !x4) || (!x2 && x6) || (!x4 && x6);
    const bool m3 = (!x3 && !x5) || (!x3 && !x6) || (!x5 && !x6);
    return (uint32_t)m0 | ((uint32_t)m1 << 1) | ((uint32_t)m2 << 2) | ((uint32_t)m3 << 3);
}

// Encoding of a keep mask (bits 0..3) into the 4-bit metadata code idx0 | idx1 << 2.  The same
// boolean formulas serve masks with fewer or more than two bits (fall-back encodings).
__device__ __forceinline__ uint32_t encode_nibble(uint32_t mask) {
    const uint32_t m0 = mask & 1u, m1 = (mask >> 1) & 1u, m2 = (mask >> 2) & 1u;
    const uint32_t bit0 = (m0 ^ 1u) & m1;
    const uint32_t bit1 = (m0 ^ 1u) & (m1 ^ 1u);
    const uint32_t bit2 = bit1 | (m2 ^ 1u);
    const uint32_t bit3 = bit0 | (m1 ^ 1u) | m2;
    return bit0 | (bit1 << 1) | (bit2 << 2) | (bit3 << 3);
}

template <typename T> __device__ __forceinline__ T pick4(uint32_t idx, T v0, T v1, T v2, T v3) {
    const T lo = (idx & 1u) ? v1 : v0;
    const T hi = (idx & 1u) ? v3 : v2;
    return (idx & 2u) ? hi : lo;
}

// ---------------------------------------------------------------------------------------------
// metadata placement: logical element (r, c) of the (m, ncols) metadata matrix -> flat offset in the
// reordered buffer.  GROUP/INTER = 32/4 for 16-bit metadata words, 16/2 for 32-bit words.
// ---------------------------------------------------------------------------------------------
template <int META_BYTES> __device__ __forceinline__ int64_t meta_offset(int64_t r, int64_t c, int64_t m) {
    constexpr int GROUP = META_BYTES == 2 ? 32 : 16;
    constexpr int INTER = META_BYTES == 2 ? 4 : 2;
    int64_t dr = r / GROUP * GROUP + (r % 8) * INTER + (r % GROUP) / 8;
    int64_t dc = c;
    const bool r_odd = dr & 1, c_odd = dc & 1;
    if (!r_odd && c_odd) { dr += 1; dc -= 1; }
    else if (r_odd && !c_odd) { dr -= 1; dc += 1; }
    return (dc >> 1) * (2 * m) + dr * 2 + (dc & 1);
}

// Inside one aligned group of GROUP rows and one column pair the destination is a contiguous run of
// 2*GROUP words.  Position (0 .. 2*GROUP-1) of (row-in-group rr, column parity cp) inside that run.
template <int META_BYTES> __device__ __forceinline__ int meta_run_pos(int rr, int cp) {
    constexpr int GROUP = META_BYTES == 2 ? 32 : 16;
    constexpr int INTER = META_BYTES == 2 ? 4 : 2;
    int dr = (rr % 8) * INTER + (rr % GROUP) / 8;
    int dc = cp;
    if (!(dr & 1) && dc) { dr += 1; dc = 0; }
    else if ((dr & 1) && !dc) { dr -= 1; dc = 1; }
    return dr * 2 + dc;
}

// ---------------------------------------------------------------------------------------------
// Philox4x32-10 and the uniform pair of a group
// ---------------------------------------------------------------------------------------------
// Philox4x32 with ROUNDS rounds: 10 for the exact MVUE mode; 7 (the fewest rounds Salmon et al. report as passing
// BigCrush) for the fast mode.  The reference draws with five (tl.rand4x(..., n_rounds=5)).
template <int ROUNDS = 10> __device__ __forceinline__ uint4 philox4x32(uint4 c, uint2 k) {
    constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
    for (int i = 0; i < ROUNDS; ++i) {
        const uint32_t hi0 = __umulhi(M0, c.x), lo0 = M0 * c.x;
        const uint32_t hi1 = __umulhi(M1, c.z), lo1 = M1 * c.z;
        c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
        k.x += W0;
        k.y += W1;
    }
    return c;
}

__device__ __forceinline__ float u32_to_uniform(uint32_t x) { return (float)(x >> 8) * 5.9604644775390625e-08f; }

// Uniform pairs of the two groups 2*pair and 2*pair+1 (linear group index over the logical matrix).
template <int ROUNDS = 10>
__device__ __forceinline__ void mvue_uniform_pairs(uint64_t pair, uint64_t seed, uint64_t offset, float &u0a,
                                                   float &u1a, float &u0b, float &u1b) {
    const uint4 r = philox4x32<ROUNDS>(make_uint4((uint32_t)pair, (uint32_t)(pair >> 32), (uint32_t)offset,
                                             (uint32_t)(offset >> 32)),
                                  make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
    u0a = u32_to_uniform(r.x); u1a = u32_to_uniform(r.y);
    u0b = u32_to_uniform(r.z); u1b = u32_to_uniform(r.w);
}

// ---------------------------------------------------------------------------------------------
// MVUE24 (approximate): float32, one rounding per operation, left-to-right sums, IEEE division.
// x[] is overwritten with x_i / p_i; returns the keep mask as bits 0..3.
// ---------------------------------------------------------------------------------------------
template <bool ALL_FOUR = true>
__device__ __forceinline__ uint32_t mvue24_group(float (&x)[4], float u0, float u1) {
    const float eps = 1.19209e-07f;
    float a[4], t[4], kk[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = __fadd_rn(fabsf(x[i]), eps);
    const float s = __fadd_rn(__fadd_rn(__fadd_rn(a[0], a[1]), a[2]), a[3]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        t[i] = __fdiv_rn(a[i], s);
        kk[i] = __fdiv_rn(t[i], __fsub_rn(s, a[i]));
    }
    const float ks = __fadd_rn(__fadd_rn(__fadd_rn(kk[0], kk[1]), kk[2]), kk[3]);
    const float t01 = __fadd_rn(t[0], t[1]);
    const float t012 = __fadd_rn(t01, t[2]);
    const bool m0 = u0 <= t[0];
    const bool m1 = (u0 <= t01) && !m0;
    const bool m2 = (u0 <= t012) && !m1 && !m0;
    const bool m3 = !m2 && !m1 && !m0;
    // (~m) * a : 0 * a when picked (NaN for an infinite a, like the reference), 1 * a otherwise
    const float d0 = __fmul_rn(m0 ? 0.f : 1.f, a[0]);
    const float d1 = __fmul_rn(m1 ? 0.f : 1.f, a[1]);
    const float d2 = __fmul_rn(m2 ? 0.f : 1.f, a[2]);
    const float d3 = __fmul_rn(m3 ? 0.f : 1.f, a[3]);
    const float d01 = __fadd_rn(d0, d1);
    const float d012 = __fadd_rn(d01, d2);
    const float ds = __fadd_rn(d012, d3);
    const float tt = __fmul_rn(u1, ds);
    const bool e0 = tt <= d0;
    const bool e1 = (tt <= d01) && !e0;
    const bool e2 = (tt <= d012) && !e1 && !e0;
    const bool e3 = !e2 && !e1 && !e0;
    const uint32_t keep = (uint32_t)(m0 || e0) | ((uint32_t)(m1 || e1) << 1) | ((uint32_t)(m2 || e2) << 2) |
                          ((uint32_t)(m3 || e3) << 3);
    if constexpr (ALL_FOUR) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float p = __fadd_rn(t[i], __fmul_rn(a[i], __fsub_rn(ks, kk[i])));
            x[i] = __fdiv_rn(x[i], p);
        }
    } else {
        // compressed output: only the two stored positions are divided (the same two quotients the full form
        // would pick); they come back in x[0], x[1]
        float p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = __fadd_rn(t[i], __fmul_rn(a[i], __fsub_rn(ks, kk[i])));
        const uint32_t nib = encode_nibble(keep);
        const float q0 = __fdiv_rn(pick4(nib & 3u, x[0], x[1], x[2], x[3]), pick4(nib & 3u, p[0], p[1], p[2], p[3]));
        const float q1 = __fdiv_rn(pick4(nib >> 2, x[0], x[1], x[2], x[3]), pick4(nib >> 2, p[0], p[1], p[2], p[3]));
        x[0] = q0;
        x[1] = q1;
    }
    return keep;
}

// ---------------------------------------------------------------------------------------------
// MVUE24, fast arithmetic (seeded mode only).  The same estimator - sample two of four without replacement with
// probability proportional to a_i = |x_i| + eps, store x_i / p_i with p_i the inclusion probability - arranged for
// the instruction mix of the SM instead of for bit-equality with the reference formulas:
//   * every division is a reciprocal approximation (MUFU) and a multiply;
//   * S - a_i and K - k_i are taken as the sum of the other three terms, not as a difference: no cancellation when one
//     magnitude dominates its group, so p_i is good to a few float32 ulps everywhere (the reference order loses up to
//     ~1e-4 relative there);
//   * a draw is a count of thresholds below the scaled uniform instead of a cascade of dependent predicates;
//   * all four quotients are formed (two more reciprocals) so that the two stored ones can be gathered with one
//     table-driven byte permute instead of select chains.
// Every operation is an explicit intrinsic (no compiler contraction), so all kernels that call this function produce
// the same bits for the same inputs.  As in the reference, a second uniform of exactly zero repeats a first pick of
// position 0 (one kept value in that group, probability ~2^-25).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float rcp_fast(float v) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}
constexpr int kMvueFastRounds = 7;

// 23 random bits -> float32 uniform on [0, 1) with 2^-23 spacing (mantissa of a float in [1, 2), minus one)
__device__ __forceinline__ float u32_to_uniform23(uint32_t x) {
    return __fadd_rn(__uint_as_float((x & 0x007FFFFFu) | 0x3F800000u), -1.f);
}

// Uniform pairs of groups 2*pair and 2*pair+1 for the fast mode: Philox4x32-7, 23-bit uniforms.
__device__ __forceinline__ void mvue_uniform_pairs_fast(uint64_t pair, uint64_t seed, uint64_t offset, float &u0a,
                                                        float &u1a, float &u0b, float &u1b) {
    const uint4 r = philox4x32<kMvueFastRounds>(make_uint4((uint32_t)pair, (uint32_t)(pair >> 32), (uint32_t)offset,
                                                           (uint32_t)(offset >> 32)),
                                                make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
    u0a = u32_to_uniform23(r.x); u1a = u32_to_uniform23(r.y);
    u0b = u32_to_uniform23(r.z); u1b = u32_to_uniform23(r.w);
}

// number of thresholds c0 <= c1 <= c2 strictly below w: 0..3
__device__ __forceinline__ uint32_t count_below(float w, float c0, float c1, float c2) {
    return (uint32_t)(w > c0) + (uint32_t)(w > c1) + (uint32_t)(w > c2);
}

// x[] is overwritten with x_i / p_i for ALL four positions; returns the keep mask as bits 0..3.
__device__ __forceinline__ uint32_t mvue24_group_fast(float (&x)[4], float u0, float u1) {
    const float eps = 1.19209e-07f;
    const float a0 = __fadd_rn(fabsf(x[0]), eps), a1 = __fadd_rn(fabsf(x[1]), eps);
    const float a2 = __fadd_rn(fabsf(x[2]), eps), a3 = __fadd_rn(fabsf(x[3]), eps);
    const float a01 = __fadd_rn(a0, a1), a23 = __fadd_rn(a2, a3);
    const float s = __fadd_rn(a01, a23), a012 = __fadd_rn(a01, a2);
    // sums of the other three
    const float s0 = __fadd_rn(a1, a23), s1 = __fadd_rn(a0, a23), s2 = __fadd_rn(a01, a3);
    const float rs = rcp_fast(s);
    const float t0 = __fmul_rn(a0, rs), t1 = __fmul_rn(a1, rs), t2 = __fmul_rn(a2, rs), t3 = __fmul_rn(a3, rs);
    const float k0 = __fmul_rn(t0, rcp_fast(s0)), k1 = __fmul_rn(t1, rcp_fast(s1));
    const float k2 = __fmul_rn(t2, rcp_fast(s2)), k3 = __fmul_rn(t3, rcp_fast(a012));
    const float k01 = __fadd_rn(k0, k1), k23 = __fadd_rn(k2, k3);
    const float p0 = __fmaf_rn(a0, __fadd_rn(k1, k23), t0), p1 = __fmaf_rn(a1, __fadd_rn(k0, k23), t1);
    const float p2 = __fmaf_rn(a2, __fadd_rn(k01, k3), t2), p3 = __fmaf_rn(a3, __fadd_rn(k01, k2), t3);
    // first pick: the interval of the cumulative sums (a0, a01, a012, s) that u0 * s falls into
    const float w = __fmul_rn(u0, s);
    const bool b0 = w > a0, b2 = w > a012;
    const uint32_t f = (uint32_t)b0 + (uint32_t)(w > a01) + (uint32_t)b2;
    // second pick among the other three: the same walk over the cumulative sums with the first pick's weight zeroed
    const float d0 = b0 ? a0 : 0.f, d1 = f == 1u ? 0.f : a1, d2 = f == 2u ? 0.f : a2, d3 = b2 ? 0.f : a3;
    const float d01 = __fadd_rn(d0, d1), d012 = __fadd_rn(d01, d2);
    const uint32_t g = count_below(__fmul_rn(u1, __fadd_rn(d012, d3)), d0, d01, d012);
    x[0] = __fmul_rn(x[0], rcp_fast(p0));
    x[1] = __fmul_rn(x[1], rcp_fast(p1));
    x[2] = __fmul_rn(x[2], rcp_fast(p2));
    x[3] = __fmul_rn(x[3], rcp_fast(p3));
    return (1u << f) | (1u << g);
}

// ---------------------------------------------------------------------------------------------
// host-side helpers
// ---------------------------------------------------------------------------------------------
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int dtype_size(int dt) {
    switch (dt) {
        case SP24_F32: return 4;
        case SP24_F16: case SP24_BF16: return 2;
        case SP24_E4M3: case SP24_E5M2: case SP24_I8: return 1;
        case SP24_I32: return 4;
        default: return 0;
    }
}
int check_device();            // SP24_OK when the current device is compute capability 10.x
int launch_status();           // maps cudaGetLastError() to SP24_OK / SP24_ERR_CUDA
int sm_count();                // SMs of the current device

}  // namespace sp24
