// Dense-shaped 2:4 prune ops (MVUE24, magnitude prune, S-STE soft threshold), 2:4 -> dense
// decompression and the masked-decay update.  All are streaming HBM-bound kernels built on
// 16-byte coalesced accesses; every output element is written by the kernel (no memset pass).
#include "sp24_common.cuh"

namespace sp24 {
namespace {

enum { OP_MVUE = 0, OP_SPARSE24 = 1, OP_SOFT = 2, OP_MVUE_FAST = 3 };
constexpr bool op_is_mvue(int op) { return op == OP_MVUE || op == OP_MVUE_FAST; }

struct DenseParams {
    const void *x;
    void *sparse;
    void *mask;
    const float *uniforms;
    int64_t m, k, ld_x, ld_s, ld_m, ld_u;
    uint64_t seed, offset;
    float scale;
    int use_scale;
};

// One group of four.  in[] are the stored elements; s[] / mk[] receive the outputs.
template <typename T, int OP>
__device__ __forceinline__ void dense_group(const T (&in)[4], float u0, float u1, const DenseParams &P, T (&s)[4],
                                            T (&mk)[4]) {
    const T zero = Elem<T>::from_f32(0.f), one = Elem<T>::from_f32(1.f);
    float x[4] = {Elem<T>::to_f32(in[0]), Elem<T>::to_f32(in[1]), Elem<T>::to_f32(in[2]), Elem<T>::to_f32(in[3])};
    if constexpr (op_is_mvue(OP)) {
        uint32_t keep;
        if constexpr (OP == OP_MVUE) keep = mvue24_group(x, u0, u1);
        else keep = mvue24_group_fast(x, u0, u1);
#pragma unroll
        for (int i = 0; i < 4; ++i) s[i] = ((keep >> i) & 1u) ? Elem<T>::from_f32(x[i]) : zero;
    } else {
        const uint32_t keep = magnitude_mask4(x[0], x[1], x[2], x[3]);
        if constexpr (OP == OP_SPARSE24) {
#pragma unroll
            for (int i = 0; i < 4; ++i) s[i] = ((keep >> i) & 1u) ? in[i] : zero;
        } else {
            const float a0 = fabsf(x[0]), a1 = fabsf(x[1]), a2 = fabsf(x[2]), a3 = fabsf(x[3]);
            const float thr = fminf(fmaxf(fminf(a0, a1), fminf(a2, a3)), fminf(fmaxf(a0, a1), fmaxf(a2, a3)));
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                T v = Elem<T>::from_f32(x[i] > 0.f ? __fsub_rn(x[i], thr) : __fadd_rn(x[i], thr));
                if (P.use_scale) v = Elem<T>::from_f32(__fmul_rn(Elem<T>::to_f32(v), P.scale));
                s[i] = ((keep >> i) & 1u) ? v : zero;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) mk[i] = ((keep >> i) & 1u) ? one : zero;
    }
}

// row-major: one item = 8 consecutive elements of a row (two groups, one Philox block).
template <typename T, int OP, bool HAS_U> __global__ void __launch_bounds__(256) dense_row_kernel(DenseParams P) {
    constexpr int ITEMS = 2;
    const int64_t per_row = P.k / 8;
    const int64_t total = P.m * per_row;
    const T *x = static_cast<const T *>(P.x);
    T *sp = static_cast<T *>(P.sparse);
    T *mo = static_cast<T *>(P.mask);
    const int64_t base = (int64_t)blockIdx.x * (256 * ITEMS) + threadIdx.x;
    T in[ITEMS][8];
    int64_t rr[ITEMS], cc[ITEMS];
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        const int64_t idx = base + it * 256;
        // 64-bit division is emulated (dozens of instructions); matrices below 2^31 items take the 32-bit one
        if (total <= 0x7FFFFFFF) rr[it] = (int64_t)((uint32_t)idx / (uint32_t)per_row);
        else rr[it] = idx / per_row;
        cc[it] = (idx - rr[it] * per_row) * 8;
        if (idx < total) {
            T tmp[8];
#pragma unroll
            for (int v = 0; v < (int)(8 * sizeof(T) / 16); ++v) {
                constexpr int PER = 16 / sizeof(T);
                Vec<T, PER> vv = load_vec<T, PER>(x + rr[it] * P.ld_x + cc[it] + v * PER);
#pragma unroll
                for (int j = 0; j < PER; ++j) tmp[v * PER + j] = vv.v[j];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) in[it][j] = tmp[j];
        }
    }
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        const int64_t idx = base + it * 256;
        if (idx >= total) continue;
        float u[4] = {0.f, 0.f, 0.f, 0.f};
        if constexpr (op_is_mvue(OP)) {
            if constexpr (HAS_U) {
                const float *up = P.uniforms + rr[it] * P.ld_u + cc[it];
                const float2 ua = *reinterpret_cast<const float2 *>(up);
                const float2 ub = *reinterpret_cast<const float2 *>(up + 4);
                u[0] = ua.x; u[1] = ua.y; u[2] = ub.x; u[3] = ub.y;
            } else {
                const uint64_t gi = (uint64_t)rr[it] * (uint64_t)(P.k / 4) + (uint64_t)(cc[it] / 4);
                if constexpr (OP == OP_MVUE_FAST) mvue_uniform_pairs_fast(gi >> 1, P.seed, P.offset, u[0], u[1], u[2], u[3]);
                else mvue_uniform_pairs(gi >> 1, P.seed, P.offset, u[0], u[1], u[2], u[3]);
            }
        }
        T s[8], mk[8];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const T grp[4] = {in[it][4 * h], in[it][4 * h + 1], in[it][4 * h + 2], in[it][4 * h + 3]};
            T so[4], mo4[4];
            dense_group<T, OP>(grp, u[2 * h], u[2 * h + 1], P, so, mo4);
#pragma unroll
            for (int i = 0; i < 4; ++i) { s[4 * h + i] = so[i]; if constexpr (!op_is_mvue(OP)) mk[4 * h + i] = mo4[i]; }
        }
        constexpr int PER = 16 / sizeof(T);
#pragma unroll
        for (int v = 0; v < 8 / PER; ++v) {
            Vec<T, PER> vs, vm;
#pragma unroll
            for (int j = 0; j < PER; ++j) { vs.v[j] = s[v * PER + j]; if constexpr (!op_is_mvue(OP)) vm.v[j] = mk[v * PER + j]; }
            store_vec<T, PER>(sp + rr[it] * P.ld_s + cc[it] + v * PER, vs);
            if constexpr (!op_is_mvue(OP)) store_vec<T, PER>(mo + rr[it] * P.ld_m + cc[it] + v * PER, vm);
        }
    }
}

// column-major storage: element (r, c) at c*ld + r; thread = V consecutive r x 8 storage rows.
template <typename T, int OP, bool HAS_U> __global__ void __launch_bounds__(256) dense_col_kernel(DenseParams P) {
    constexpr int V = 16 / sizeof(T);
    const int64_t r = ((int64_t)blockIdx.x * 256 + threadIdx.x) * V;
    const int64_t c8 = (int64_t)blockIdx.y * 8;
    if (r >= P.m) return;
    const T *x = static_cast<const T *>(P.x);
    T *sp = static_cast<T *>(P.sparse);
    T *mo = static_cast<T *>(P.mask);
    Vec<T, V> in[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) in[j] = load_vec<T, V>(x + (c8 + j) * P.ld_x + r);
    float u[V][4];
    if constexpr (op_is_mvue(OP)) {
        if constexpr (HAS_U) {
            constexpr int FV = 4;
#pragma unroll
            for (int q = 0; q < V / FV; ++q) {
                const Vec<float, FV> t0 = load_vec<float, FV>(P.uniforms + (c8 + 0) * P.ld_u + r + q * FV);
                const Vec<float, FV> t1 = load_vec<float, FV>(P.uniforms + (c8 + 1) * P.ld_u + r + q * FV);
                const Vec<float, FV> t2 = load_vec<float, FV>(P.uniforms + (c8 + 4) * P.ld_u + r + q * FV);
                const Vec<float, FV> t3 = load_vec<float, FV>(P.uniforms + (c8 + 5) * P.ld_u + r + q * FV);
#pragma unroll
                for (int j = 0; j < FV; ++j) {
                    u[q * FV + j][0] = t0.v[j]; u[q * FV + j][1] = t1.v[j];
                    u[q * FV + j][2] = t2.v[j]; u[q * FV + j][3] = t3.v[j];
                }
            }
        } else {
#pragma unroll
            for (int v = 0; v < V; ++v) {
                const uint64_t gi = (uint64_t)(r + v) * (uint64_t)(P.k / 4) + (uint64_t)(c8 / 4);
                if constexpr (OP == OP_MVUE_FAST) mvue_uniform_pairs_fast(gi >> 1, P.seed, P.offset, u[v][0], u[v][1], u[v][2], u[v][3]);
                else mvue_uniform_pairs(gi >> 1, P.seed, P.offset, u[v][0], u[v][1], u[v][2], u[v][3]);
            }
        }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        Vec<T, V> so[4], mk[4];
#pragma unroll
        for (int v = 0; v < V; ++v) {
            const T grp[4] = {in[4 * h].v[v], in[4 * h + 1].v[v], in[4 * h + 2].v[v], in[4 * h + 3].v[v]};
            T s4[4], m4[4];
            float ua = 0.f, ub = 0.f;
            if constexpr (op_is_mvue(OP)) { ua = u[v][2 * h]; ub = u[v][2 * h + 1]; }
            dense_group<T, OP>(grp, ua, ub, P, s4, m4);
#pragma unroll
            for (int i = 0; i < 4; ++i) { so[i].v[v] = s4[i]; if constexpr (!op_is_mvue(OP)) mk[i].v[v] = m4[i]; }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            store_vec<T, V>(sp + (c8 + 4 * h + i) * P.ld_s + r, so[i]);
            if constexpr (!op_is_mvue(OP)) store_vec<T, V>(mo + (c8 + 4 * h + i) * P.ld_m + r, mk[i]);
        }
    }
}

template <typename T, int OP, bool HAS_U> int launch_dense(const DenseParams &P, int col_major, cudaStream_t st) {
    if (!col_major) {
        const int64_t total = P.m * (P.k / 8);
        dense_row_kernel<T, OP, HAS_U><<<(unsigned)((total + 511) / 512), 256, 0, st>>>(P);
    } else {
        constexpr int V = 16 / sizeof(T);
        dim3 grid((unsigned)((P.m / V + 255) / 256), (unsigned)(P.k / 8));
        dense_col_kernel<T, OP, HAS_U><<<grid, 256, 0, st>>>(P);
    }
    return launch_status();
}

template <int OP> int dispatch_dense(const DenseParams &P, int dtype, int col_major, cudaStream_t st) {
    const bool has_u = P.uniforms != nullptr;
    switch (dtype) {
        case SP24_F32:
            return has_u ? launch_dense<float, OP, true>(P, col_major, st) : launch_dense<float, OP, false>(P, col_major, st);
        case SP24_F16:
            return has_u ? launch_dense<__half, OP, true>(P, col_major, st)
                         : launch_dense<__half, OP, false>(P, col_major, st);
        case SP24_BF16:
            return has_u ? launch_dense<__nv_bfloat16, OP, true>(P, col_major, st)
                         : launch_dense<__nv_bfloat16, OP, false>(P, col_major, st);
        default: return SP24_ERR_DTYPE;
    }
}

int check_dense_args(const void *x, int dtype, int64_t m, int64_t k, int64_t ld_x, int col_major, const void *o1,
                     int64_t ld1, const void *o2, int64_t ld2, bool need_o2) {
    if (!x || !o1 || (need_o2 && !o2)) return SP24_ERR_ARG;
    const int sz = dtype_size(dtype);
    if (dtype != SP24_F32 && dtype != SP24_F16 && dtype != SP24_BF16) return SP24_ERR_DTYPE;
    const int64_t v = 16 / sz;
    if (m <= 0 || k <= 0 || k % 8) return SP24_ERR_SHAPE;
    if (col_major && m % v) return SP24_ERR_SHAPE;
    const int64_t inner = col_major ? m : k;
    if (ld_x < inner || ld_x % v || ld1 < inner || ld1 % v || (need_o2 && (ld2 < inner || ld2 % v))) return SP24_ERR_STRIDE;
    if (!aligned16(x) || !aligned16(o1) || (need_o2 && !aligned16(o2))) return SP24_ERR_ALIGN;
    return check_device();
}

// ---------------------------------------------------------------------------------------------
// 2:4 -> dense.  Thread = one metadata word: CH/2 packed values in, CH dense elements out.
// ---------------------------------------------------------------------------------------------
template <typename T> __global__ void __launch_bounds__(256) to_dense_kernel(const T *packed, const void *meta, T *dense,
                                                                              int64_t m, int64_t k, int64_t ld_p,
                                                                              int64_t ld_d) {
    constexpr int CH = sizeof(T) == 2 ? 16 : 32;
    constexpr int MB = sizeof(T) == 2 ? 2 : 4;
    using MetaT = typename VecBytes<MB>::type;
    const int64_t ncols = k / CH;
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (idx >= m * ncols) return;
    const int64_t r = idx / ncols, c = idx - r * ncols;
    const uint32_t word = (uint32_t) static_cast<const MetaT *>(meta)[meta_offset<MB>(r, c, m)];
    T vals[CH / 2];
    {
        Vec<T, CH / 2> v = load_vec<T, CH / 2>(packed + r * ld_p + c * (CH / 2));
#pragma unroll
        for (int j = 0; j < CH / 2; ++j) vals[j] = v.v[j];
    }
    T out[CH];
    T zero;
    memset(&zero, 0, sizeof(T));
#pragma unroll
    for (int g = 0; g < CH / 4; ++g) {
        const uint32_t nib = (word >> (4 * g)) & 0xFu;
        const uint32_t i0 = nib & 3u, i1 = nib >> 2;
#pragma unroll
        for (int i = 0; i < 4; ++i) out[4 * g + i] = zero;
        // same order as a scatter of value 0 then value 1 (the later write wins when both indices coincide)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (i0 == (uint32_t)i) out[4 * g + i] = vals[2 * g];
            if (i1 == (uint32_t)i) out[4 * g + i] = vals[2 * g + 1];
        }
    }
    constexpr int PER = 16 / sizeof(T);
#pragma unroll
    for (int v = 0; v < CH / PER; ++v) {
        Vec<T, PER> vv;
#pragma unroll
        for (int j = 0; j < PER; ++j) vv.v[j] = out[v * PER + j];
        store_vec<T, PER>(dense + r * ld_d + c * CH + v * PER, vv);
    }
}

// ---------------------------------------------------------------------------------------------
// masked decay: grad[i] += p[i] * alpha where mask[i] == 0.  Four elements per thread and pass.
// ---------------------------------------------------------------------------------------------
template <int MS> __device__ __forceinline__ uint32_t load_keep4(const void *mask, int64_t i) {
    if constexpr (MS == 1) {
        const uint32_t w = *reinterpret_cast<const uint32_t *>(static_cast<const uint8_t *>(mask) + i);
        return ((w & 0xFFu) != 0) | (((w >> 8) & 0xFFu) != 0) << 1 | (((w >> 16) & 0xFFu) != 0) << 2 | ((w >> 24) != 0) << 3;
    } else if constexpr (MS == 2) {
        const uint2 w = *reinterpret_cast<const uint2 *>(static_cast<const uint16_t *>(mask) + i);
        return ((w.x & 0x7FFFu) != 0) | (((w.x >> 16) & 0x7FFFu) != 0) << 1 | ((w.y & 0x7FFFu) != 0) << 2 |
               (((w.y >> 16) & 0x7FFFu) != 0) << 3;
    } else {
        const uint4 w = *reinterpret_cast<const uint4 *>(static_cast<const uint32_t *>(mask) + i);
        return ((w.x & 0x7FFFFFFFu) != 0) | ((w.y & 0x7FFFFFFFu) != 0) << 1 | ((w.z & 0x7FFFFFFFu) != 0) << 2 |
               ((w.w & 0x7FFFFFFFu) != 0) << 3;
    }
}

template <int MS>
__global__ void __launch_bounds__(256) masked_add_kernel(float *grad, const float *p, const void *mask, int64_t n,
                                                         float alpha) {
    constexpr int UNR = 4;
    const int64_t n4 = n / 4;
    const int64_t base = (int64_t)blockIdx.x * (256 * UNR) + threadIdx.x;
    float4 g[UNR], q[UNR];
    uint32_t keep[UNR];
#pragma unroll
    for (int j = 0; j < UNR; ++j) {
        const int64_t i = base + j * 256;
        if (i < n4) {
            keep[j] = load_keep4<MS>(mask, i * 4);
            g[j] = reinterpret_cast<const float4 *>(grad)[i];
            q[j] = reinterpret_cast<const float4 *>(p)[i];
        }
    }
#pragma unroll
    for (int j = 0; j < UNR; ++j) {
        const int64_t i = base + j * 256;
        if (i < n4 && keep[j] != 0xFu) {
            if (!(keep[j] & 1u)) g[j].x = __fadd_rn(g[j].x, __fmul_rn(q[j].x, alpha));
            if (!(keep[j] & 2u)) g[j].y = __fadd_rn(g[j].y, __fmul_rn(q[j].y, alpha));
            if (!(keep[j] & 4u)) g[j].z = __fadd_rn(g[j].z, __fmul_rn(q[j].z, alpha));
            if (!(keep[j] & 8u)) g[j].w = __fadd_rn(g[j].w, __fmul_rn(q[j].w, alpha));
            reinterpret_cast<float4 *>(grad)[i] = g[j];
        }
    }
    // ragged tail (n not a multiple of 4): handled by the first threads of block 0
    if (blockIdx.x == 0 && threadIdx.x < (int)(n - n4 * 4)) {
        const int64_t i = n4 * 4 + threadIdx.x;
        bool kp;
        if constexpr (MS == 1) kp = static_cast<const uint8_t *>(mask)[i] != 0;
        else if constexpr (MS == 2) kp = (static_cast<const uint16_t *>(mask)[i] & 0x7FFFu) != 0;
        else kp = (static_cast<const uint32_t *>(mask)[i] & 0x7FFFFFFFu) != 0;
        if (!kp) grad[i] = __fadd_rn(grad[i], __fmul_rn(p[i], alpha));
    }
}

}  // namespace
}  // namespace sp24

using namespace sp24;

extern "C" int sp24_mvue24_dense(const void *x, int dtype, int64_t m, int64_t k, int64_t ld_x, int col_major, void *out,
                                 int64_t ld_out, const float *uniforms, int64_t ld_uniforms, uint64_t seed,
                                 uint64_t offset, void *stream) {
    if (int rc = check_dense_args(x, dtype, m, k, ld_x, col_major, out, ld_out, nullptr, 0, false)) return rc;
    if (uniforms) {
        const int64_t inner = col_major ? m : k;
        if (ld_uniforms < inner || ld_uniforms % 4) return SP24_ERR_STRIDE;
        if (!aligned16(uniforms)) return SP24_ERR_ALIGN;
    }
    DenseParams P{x, out, nullptr, uniforms, m, k, ld_x, ld_out, 0, ld_uniforms, seed, offset, 1.f, 0};
    return dispatch_dense<OP_MVUE>(P, dtype, col_major, static_cast<cudaStream_t>(stream));
}

// The same estimator with the fast arithmetic of SP24_PRUNE_MVUE_FAST (seeded only): what the compressing kernel
// stores for (seed, offset) in that mode is what this one writes at the kept positions, bit for bit.
extern "C" int sp24_mvue24_dense_fast(const void *x, int dtype, int64_t m, int64_t k, int64_t ld_x, int col_major, void *out,
                                      int64_t ld_out, uint64_t seed, uint64_t offset, void *stream) {
    if (int rc = check_dense_args(x, dtype, m, k, ld_x, col_major, out, ld_out, nullptr, 0, false)) return rc;
    DenseParams P{x, out, nullptr, nullptr, m, k, ld_x, ld_out, 0, 0, seed, offset, 1.f, 0};
    return dispatch_dense<OP_MVUE_FAST>(P, dtype, col_major, static_cast<cudaStream_t>(stream));
}

extern "C" int sp24_sparse24(const void *x, int dtype, int64_t m, int64_t k, int64_t ld_x, int col_major, void *sparse,
                             int64_t ld_sparse, void *mask, int64_t ld_mask, void *stream) {
    if (int rc = check_dense_args(x, dtype, m, k, ld_x, col_major, sparse, ld_sparse, mask, ld_mask, true)) return rc;
    DenseParams P{x, sparse, mask, nullptr, m, k, ld_x, ld_sparse, ld_mask, 0, 0, 0, 1.f, 0};
    return dispatch_dense<OP_SPARSE24>(P, dtype, col_major, static_cast<cudaStream_t>(stream));
}

extern "C" int sp24_soft_threshold24(const void *x, int dtype, int64_t m, int64_t k, int64_t ld_x, int col_major,
                                     void *sparse, int64_t ld_sparse, void *mask, int64_t ld_mask, int use_scale,
                                     float scale, void *stream) {
    if (int rc = check_dense_args(x, dtype, m, k, ld_x, col_major, sparse, ld_sparse, mask, ld_mask, true)) return rc;
    DenseParams P{x, sparse, mask, nullptr, m, k, ld_x, ld_sparse, ld_mask, 0, 0, 0, scale, use_scale ? 1 : 0};
    return dispatch_dense<OP_SOFT>(P, dtype, col_major, static_cast<cudaStream_t>(stream));
}

extern "C" int sp24_to_dense(const void *packed, int dtype, int64_t m, int64_t k, int64_t ld_packed, const void *meta,
                             void *dense, int64_t ld_dense, void *stream) {
    if (!packed || !meta || !dense) return SP24_ERR_ARG;
    const int sz = dtype_size(dtype);
    if (sz == 0 || dtype == SP24_F32) return SP24_ERR_DTYPE;
    const int64_t kmult = sz == 2 ? 64 : 128;
    if (m <= 0 || k <= 0 || m % 32 || k % kmult) return SP24_ERR_SHAPE;
    if (ld_packed < k / 2 || (ld_packed * sz) % 16 || ld_dense < k || (ld_dense * sz) % 16) return SP24_ERR_STRIDE;
    if (!aligned16(packed) || !aligned16(meta) || !aligned16(dense)) return SP24_ERR_ALIGN;
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (sz == 2) {
        const int64_t total = m * (k / 16);
        to_dense_kernel<uint16_t><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
            static_cast<const uint16_t *>(packed), meta, static_cast<uint16_t *>(dense), m, k, ld_packed, ld_dense);
    } else {
        const int64_t total = m * (k / 32);
        to_dense_kernel<uint8_t><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
            static_cast<const uint8_t *>(packed), meta, static_cast<uint8_t *>(dense), m, k, ld_packed, ld_dense);
    }
    return launch_status();
}

extern "C" int sp24_masked_add(void *grad, const void *p, const void *mask, int mask_itemsize, int64_t n, float alpha,
                               void *stream) {
    if (!grad || !p || !mask) return SP24_ERR_ARG;
    if (n < 0) return SP24_ERR_SHAPE;
    if (n == 0) return SP24_OK;
    if (mask_itemsize != 1 && mask_itemsize != 2 && mask_itemsize != 4) return SP24_ERR_DTYPE;
    if (!aligned16(grad) || !aligned16(p) || (reinterpret_cast<uintptr_t>(mask) & (4 * mask_itemsize - 1)))
        return SP24_ERR_ALIGN;
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t n4 = n / 4;
    const unsigned blocks = (unsigned)((n4 + 1023) / 1024 > 0 ? (n4 + 1023) / 1024 : 1);
    float *g = static_cast<float *>(grad);
    const float *q = static_cast<const float *>(p);
    if (mask_itemsize == 1) masked_add_kernel<1><<<blocks, 256, 0, st>>>(g, q, mask, n, alpha);
    else if (mask_itemsize == 2) masked_add_kernel<2><<<blocks, 256, 0, st>>>(g, q, mask, n, alpha);
    else masked_add_kernel<4><<<blocks, 256, 0, st>>>(g, q, mask, n, alpha);
    return launch_status();
}

// ---------------------------------------------------------------------------------------------
// Masked decay + AdamW in one pass over a flat fp32 parameter range
// ---------------------------------------------------------------------------------------------
namespace sp24 {
namespace {

struct AdamParams {
    float *p;
    const void *g;             // gradient, float32 or 16-bit (g_dtype)
    float *m, *v;
    const uint8_t *mask;       // may be null: no masked decay
    int64_t n;
    float lr, beta1, beta2, eps, weight_decay, alpha;
    float step;                // optimizer step number (1, 2, ...) when step_dev is null
    const float *step_dev;     // optional: step number read on the device (replayed launches)
    const void *g2;            // optional second gradient, added to g on the first n2 elements (n2 % 4 == 0)
    int g2_dtype;              // SP24_F32 / SP24_F16 / SP24_BF16
    int64_t n2;
    int g_dtype;               // SP24_F32 / SP24_F16 / SP24_BF16
};

__device__ __forceinline__ float4 load_extra4(const void *g2, int dtype, int64_t i) {
    if (dtype == SP24_F32) return reinterpret_cast<const float4 *>(g2)[i];
    const uint2 r = reinterpret_cast<const uint2 *>(g2)[i];
    if (dtype == SP24_BF16)
        return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xFFFF0000u), __uint_as_float(r.y << 16),
                           __uint_as_float(r.y & 0xFFFF0000u));
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&r.x)), b = __half22float2(*reinterpret_cast<const __half2 *>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

__device__ __forceinline__ void adam_one(float &p, float g, float &m, float &v, bool keep, const AdamParams &P, float inv_bc1,
                                         float inv_sqrt_bc2) {
    // masked decay first, with the two roundings of the stand-alone kernel: grad + (p * alpha) on pruned positions
    if (!keep) g = __fadd_rn(g, __fmul_rn(p, P.alpha));
    p = p * (1.f - P.lr * P.weight_decay);
    m = m + (g - m) * (1.f - P.beta1);
    v = v * P.beta2 + (1.f - P.beta2) * g * g;
    const float denom = sqrtf(v) * inv_sqrt_bc2 + P.eps;
    p = p - (P.lr * inv_bc1) * (m / denom);
}

__global__ void __launch_bounds__(256) adamw_masked_decay_kernel(AdamParams P) {
    const float t = P.step_dev ? *P.step_dev : P.step;
    const float inv_bc1 = 1.f / (1.f - powf(P.beta1, t));
    const float inv_sqrt_bc2 = 1.f / sqrtf(1.f - powf(P.beta2, t));
    const int64_t n4 = P.n / 4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        float4 p = reinterpret_cast<const float4 *>(P.p)[i];
        float4 g = load_extra4(P.g, P.g_dtype, i);
        if (P.g2 && i * 4 < P.n2) {
            const float4 e = load_extra4(P.g2, P.g2_dtype, i);
            g = make_float4(g.x + e.x, g.y + e.y, g.z + e.z, g.w + e.w);
        }
        float4 m = reinterpret_cast<const float4 *>(P.m)[i];
        float4 v = reinterpret_cast<const float4 *>(P.v)[i];
        uint32_t mk = 0x01010101u;
        if (P.mask) mk = reinterpret_cast<const uint32_t *>(P.mask)[i];
        adam_one(p.x, g.x, m.x, v.x, (mk & 0xFFu) != 0, P, inv_bc1, inv_sqrt_bc2);
        adam_one(p.y, g.y, m.y, v.y, (mk & 0xFF00u) != 0, P, inv_bc1, inv_sqrt_bc2);
        adam_one(p.z, g.z, m.z, v.z, (mk & 0xFF0000u) != 0, P, inv_bc1, inv_sqrt_bc2);
        adam_one(p.w, g.w, m.w, v.w, (mk & 0xFF000000u) != 0, P, inv_bc1, inv_sqrt_bc2);
        reinterpret_cast<float4 *>(P.p)[i] = p;
        reinterpret_cast<float4 *>(P.m)[i] = m;
        reinterpret_cast<float4 *>(P.v)[i] = v;
    }
    // tail (n not a multiple of 4)
    const int64_t i = n4 * 4 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < P.n) {
        const bool keep = P.mask ? P.mask[i] != 0 : true;
        float g;
        if (P.g_dtype == SP24_F32) g = static_cast<const float *>(P.g)[i];
        else if (P.g_dtype == SP24_BF16) g = __bfloat162float(static_cast<const __nv_bfloat16 *>(P.g)[i]);
        else g = __half2float(static_cast<const __half *>(P.g)[i]);
        adam_one(P.p[i], g, P.m[i], P.v[i], keep, P, inv_bc1, inv_sqrt_bc2);
    }
}

}  // namespace
}  // namespace sp24

extern "C" int sp24_adamw_masked_decay_ex(void *p, const void *grad, int grad_dtype, const void *mask, void *exp_avg,
                                          void *exp_avg_sq, int64_t n, float lr, float beta1, float beta2, float eps,
                                          float weight_decay, float alpha, float step, const float *step_dev,
                                          const void *grad2, int grad2_dtype, int64_t grad2_count, void *stream) {
    using namespace sp24;
    if (!p || !grad || !exp_avg || !exp_avg_sq) return SP24_ERR_ARG;
    if (grad_dtype != SP24_F32 && grad_dtype != SP24_F16 && grad_dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (n < 0) return SP24_ERR_SHAPE;
    if (n == 0) return SP24_OK;
    if (!step_dev && !(step >= 1.f)) return SP24_ERR_ARG;
    if (grad2) {
        if (grad2_dtype != SP24_F32 && grad2_dtype != SP24_F16 && grad2_dtype != SP24_BF16) return SP24_ERR_DTYPE;
        if (grad2_count <= 0 || grad2_count > n || grad2_count % 4) return SP24_ERR_SHAPE;
    }
    if (!aligned16(p) || !aligned16(grad) || !aligned16(exp_avg) || !aligned16(exp_avg_sq) || !aligned16(grad2) ||
        (mask && (reinterpret_cast<uintptr_t>(mask) & 3u)))
        return SP24_ERR_ALIGN;
    if (int rc = check_device()) return rc;
    AdamParams P{static_cast<float *>(p), grad, static_cast<float *>(exp_avg),
                 static_cast<float *>(exp_avg_sq), static_cast<const uint8_t *>(mask), n, lr, beta1, beta2, eps, weight_decay,
                 alpha, step, step_dev, grad2, grad2_dtype, grad2 ? grad2_count : 0, grad_dtype};
    const int64_t n4 = n / 4;
    int64_t blocks = (n4 + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 16) blocks = 148 * 16;
    adamw_masked_decay_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(P);
    return launch_status();
}

extern "C" int sp24_adamw_masked_decay(void *p, const void *grad, const void *mask, void *exp_avg, void *exp_avg_sq, int64_t n,
                                       float lr, float beta1, float beta2, float eps, float weight_decay, float alpha,
                                       float step, const float *step_dev, void *stream) {
    return sp24_adamw_masked_decay_ex(p, grad, SP24_F32, mask, exp_avg, exp_avg_sq, n, lr, beta1, beta2, eps, weight_decay, alpha,
                                      step, step_dev, nullptr, 0, 0, stream);
}
