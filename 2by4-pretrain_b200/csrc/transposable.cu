// Transposable 4x4 mask select, alone and fused with the 2:4 compression of W and of W^T.
//
// One thread owns one 4x4 block.  The 90 admissible patterns (two ones per row and per column) are
// enumerated at compile time in descending lexicographic order of the row-major bit string, which is
// the nested order "row 0 pair, row 1 pair, row 2 pair, row 3 pair" over the pair list
// (0,1) (0,2) (0,3) (1,2) (1,3) (2,3).  Scores are float32 with a fixed association,
// (s0 + s1) + (s2 + s3), s_i = v[i][a] + v[i][b], and the first maximum wins.
#include "sp24_common.cuh"

namespace sp24 {
namespace {

__host__ __device__ constexpr int pair_a(int i) { return i < 3 ? 0 : (i < 5 ? 1 : 2); }
__host__ __device__ constexpr int pair_b(int i) { return i < 3 ? i + 1 : (i < 5 ? i - 1 : 3); }
__host__ __device__ constexpr int row_bits(int i) { return (1 << pair_a(i)) | (1 << pair_b(i)); }
__host__ __device__ constexpr bool cols_ok(int i0, int i1, int i2, int i3) {
    for (int c = 0; c < 4; ++c) {
        int n = 0;
        n += (pair_a(i0) == c) + (pair_b(i0) == c);
        n += (pair_a(i1) == c) + (pair_b(i1) == c);
        n += (pair_a(i2) == c) + (pair_b(i2) == c);
        n += (pair_a(i3) == c) + (pair_b(i3) == c);
        if (n != 2) return false;
    }
    return true;
}

template <int I0, int I1, int I2, int I3> struct PatternStep {
    __device__ static __forceinline__ void run(const float (&s)[4][6], float &best, uint32_t &bits) {
        if constexpr (cols_ok(I0, I1, I2, I3)) {
            const float sc = __fadd_rn(__fadd_rn(s[0][I0], s[1][I1]), __fadd_rn(s[2][I2], s[3][I3]));
            constexpr uint32_t B = row_bits(I0) | (row_bits(I1) << 4) | (row_bits(I2) << 8) | (row_bits(I3) << 12);
            if (sc > best) { best = sc; bits = B; }
        }
    }
};

// Two nested compile-time loops (36 x 36 candidates, 90 survive the column check), kept shallow so
// that the template recursion depth stays small.
template <int I0, int I1, int N> struct InnerLoop {
    __device__ static __forceinline__ void run(const float (&s)[4][6], float &best, uint32_t &bits) {
        InnerLoop<I0, I1, N - 1>::run(s, best, bits);
        PatternStep<I0, I1, (N - 1) / 6, (N - 1) % 6>::run(s, best, bits);
    }
};
template <int I0, int I1> struct InnerLoop<I0, I1, 0> {
    __device__ static __forceinline__ void run(const float (&)[4][6], float &, uint32_t &) {}
};
template <int N> struct OuterLoop {
    __device__ static __forceinline__ void run(const float (&s)[4][6], float &best, uint32_t &bits) {
        OuterLoop<N - 1>::run(s, best, bits);
        InnerLoop<(N - 1) / 6, (N - 1) % 6, 36>::run(s, best, bits);
    }
};
template <> struct OuterLoop<0> {
    __device__ static __forceinline__ void run(const float (&)[4][6], float &, uint32_t &) {}
};

// v: the 4x4 block (already |.| when requested).  Returns the 16-bit pattern, bit 4*i+j = keep (i, j).
__device__ __forceinline__ uint32_t select_pattern(const float (&v)[4][4]) {
    float s[4][6];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int p = 0; p < 6; ++p) s[i][p] = __fadd_rn(v[i][pair_a(p)], v[i][pair_b(p)]);
    float best = -INFINITY;
    // pattern 0 stays when no score compares greater than -inf (all NaN / -inf)
    uint32_t bits = row_bits(0) | (row_bits(0) << 4) | (row_bits(5) << 8) | (row_bits(5) << 12);
    OuterLoop<36>::run(s, best, bits);
    return bits;
}

template <typename T> __device__ __forceinline__ void load_row4(const T *p, T (&out)[4]) {
    Vec<T, 4> v = load_vec<T, 4>(p);
#pragma unroll
    for (int j = 0; j < 4; ++j) out[j] = v.v[j];
}

// ---------------------------------------------------------------------------------------------
// select only: x -> (sparse, mask)
// block = 8 warps = 8 block-rows (32 rows) x 32 block-columns (128 columns)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) ts_select_kernel(const T *x, T *sparse, uint8_t *mask, int64_t k, int64_t ld_x,
                                                        int64_t ld_s, int64_t ld_m, int use_abs) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t r = (int64_t)blockIdx.y * 32 + warp * 4;
    const int64_t c = (int64_t)blockIdx.x * 128 + lane * 4;
    if (c >= k) return;
    T w[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) load_row4<T>(x + (r + i) * ld_x + c, w[i]);
    float v[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float f = Elem<T>::to_f32(w[i][j]);
            v[i][j] = use_abs ? fabsf(f) : f;
        }
    const uint32_t bits = select_pattern(v);
    const T zero = Elem<T>::from_f32(0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t rb = (bits >> (4 * i)) & 0xFu;
        const uint32_t mword = (rb & 1u) | ((rb & 2u) << 7) | ((rb & 4u) << 14) | ((rb & 8u) << 21);
        *reinterpret_cast<uint32_t *>(mask + (r + i) * ld_m + c) = mword;
        if (sparse) {
            Vec<T, 4> o;
#pragma unroll
            for (int j = 0; j < 4; ++j) o.v[j] = ((rb >> j) & 1u) ? w[i][j] : zero;
            store_vec<T, 4>(sparse + (r + i) * ld_s + c, o);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// select (or read mask) + compress W and W^T.  Same thread mapping as above.
// ---------------------------------------------------------------------------------------------
struct DualParams {
    const void *w;
    uint8_t *mask;
    void *packed_w, *packed_t;
    int16_t *meta_w, *meta_t;
    int64_t m, k, ld_w, ld_mask, ld_pw, ld_pt;
};

template <typename T, typename TOut, bool SELECT>
__global__ void __launch_bounds__(256) ts_dual_kernel(DualParams P) {
    __shared__ __align__(16) uint16_t smeta_w[4][64];   // 4 column pairs x (32 rows x 2)
    __shared__ __align__(16) uint16_t smeta_t[256];     // 1 column pair x (128 rows x 2)
    __shared__ __align__(4) uint8_t nib_t[128][8];      // [W column][block row]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t r0 = (int64_t)blockIdx.y * 32, c0 = (int64_t)blockIdx.x * 128;
    const int64_t r = r0 + warp * 4, c = c0 + lane * 4;
    const bool active = c < P.k;
    const T *w_ptr = static_cast<const T *>(P.w);
    TOut *pw = static_cast<TOut *>(P.packed_w);
    TOut *pt = static_cast<TOut *>(P.packed_t);

    uint32_t bits = 0;
    T w[4][4];
    if (active) {
#pragma unroll
        for (int i = 0; i < 4; ++i) load_row4<T>(w_ptr + (r + i) * P.ld_w + c, w[i]);
        if constexpr (SELECT) {
            float v[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) v[i][j] = fabsf(Elem<T>::to_f32(w[i][j]));
            bits = select_pattern(v);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t rb = (bits >> (4 * i)) & 0xFu;
                *reinterpret_cast<uint32_t *>(P.mask + (r + i) * P.ld_mask + c) =
                    (rb & 1u) | ((rb & 2u) << 7) | ((rb & 4u) << 14) | ((rb & 8u) << 21);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t mw = *reinterpret_cast<const uint32_t *>(P.mask + (r + i) * P.ld_mask + c);
                const uint32_t rb = ((mw & 0xFFu) != 0) | (((mw >> 8) & 0xFFu) != 0) << 1 | (((mw >> 16) & 0xFFu) != 0) << 2 |
                                    ((mw >> 24) != 0) << 3;
                bits |= rb << (4 * i);
            }
        }
    }
    // rows of W: one nibble per row, four horizontally adjacent lanes make one 16-bit word
    uint32_t nib_row[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t rb = (bits >> (4 * i)) & 0xFu;
        const uint32_t nib = encode_nibble(rb);
        nib_row[i] = nib;
        if (active) {
            Vec<TOut, 2> o;
            o.v[0] = convert<TOut>(pick4(nib & 3u, w[i][0], w[i][1], w[i][2], w[i][3]));
            o.v[1] = convert<TOut>(pick4(nib >> 2, w[i][0], w[i][1], w[i][2], w[i][3]));
            store_vec<TOut, 2>(pw + (r + i) * P.ld_pw + (c >> 1), o);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t word = nib_row[i] << (4 * (lane & 3));
        word |= __shfl_xor_sync(0xFFFFFFFFu, word, 1);
        word |= __shfl_xor_sync(0xFFFFFFFFu, word, 2);
        if ((lane & 3) == 0) {
            const int mc = lane >> 2;  // metadata column inside the tile (0..7)
            smeta_w[mc >> 1][meta_run_pos<2>(warp * 4 + i, mc & 1)] = (uint16_t)word;
        }
    }
    // columns of W (= rows of W^T): one nibble per column
    {
        Vec<TOut, 4> o0, o1;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t cb = ((bits >> j) & 1u) | (((bits >> (4 + j)) & 1u) << 1) | (((bits >> (8 + j)) & 1u) << 2) |
                                (((bits >> (12 + j)) & 1u) << 3);
            const uint32_t nib = encode_nibble(cb);
            nib_t[lane * 4 + j][warp] = (uint8_t)nib;
            if (active) {
                o0.v[j] = convert<TOut>(pick4(nib & 3u, w[0][j], w[1][j], w[2][j], w[3][j]));
                o1.v[j] = convert<TOut>(pick4(nib >> 2, w[0][j], w[1][j], w[2][j], w[3][j]));
            }
        }
        if (active) {
            store_vec<TOut, 4>(pt + (r >> 1) * P.ld_pt + c, o0);
            store_vec<TOut, 4>(pt + ((r >> 1) + 1) * P.ld_pt + c, o1);
        }
    }
    __syncthreads();
    {
        // thread t: W column t>>1, metadata column parity t&1 of the transposed matrix
        const int col = threadIdx.x >> 1, par = threadIdx.x & 1;
        const uint32_t b4 = *reinterpret_cast<const uint32_t *>(&nib_t[col][par * 4]);
        const uint32_t word = (b4 & 0xFu) | ((b4 >> 4) & 0xF0u) | ((b4 >> 8) & 0xF00u) | ((b4 >> 12) & 0xF000u);
        smeta_t[(col / 32) * 64 + meta_run_pos<2>(col % 32, par)] = (uint16_t)word;
    }
    __syncthreads();
    // write-out: W metadata 4 pairs x 128 B, W^T metadata up to 512 B
    if (threadIdx.x < 32) {
        const int pair = threadIdx.x >> 3, piece = threadIdx.x & 7;
        const int64_t cp = c0 / 32 + pair;
        if (cp * 2 < P.k / 16) {
            char *dst = reinterpret_cast<char *>(P.meta_w) + (cp * 2 * P.m + 2 * r0) * 2 + piece * 16;
            *reinterpret_cast<uint4 *>(dst) =
                *reinterpret_cast<const uint4 *>(reinterpret_cast<const char *>(&smeta_w[pair][0]) + piece * 16);
        }
    } else if (threadIdx.x < 64) {
        const int piece = threadIdx.x - 32;
        const int64_t cols_here = (P.k - c0 < 128) ? (P.k - c0) : 128;
        if (piece * 8 < cols_here * 2) {
            const int64_t cp = r0 / 32;  // column pair of the (k, m) metadata matrix
            char *dst = reinterpret_cast<char *>(P.meta_t) + (cp * 2 * P.k + 2 * c0) * 2 + piece * 16;
            *reinterpret_cast<uint4 *>(dst) =
                *reinterpret_cast<const uint4 *>(reinterpret_cast<const char *>(smeta_t) + piece * 16);
        }
    }
}

template <typename T, typename TOut> int launch_dual(const DualParams &P, int select, cudaStream_t st) {
    dim3 grid((unsigned)((P.k + 127) / 128), (unsigned)(P.m / 32));
    if (select) ts_dual_kernel<T, TOut, true><<<grid, 256, 0, st>>>(P);
    else ts_dual_kernel<T, TOut, false><<<grid, 256, 0, st>>>(P);
    return launch_status();
}

template <typename T> int dispatch_dual(const DualParams &P, int packed_dtype, int select, cudaStream_t st) {
    if (packed_dtype == SP24_F16) return launch_dual<T, __half>(P, select, st);
    if (packed_dtype == SP24_BF16) return launch_dual<T, __nv_bfloat16>(P, select, st);
    return SP24_ERR_DTYPE;
}

}  // namespace
}  // namespace sp24

using namespace sp24;

extern "C" int sp24_transposable_select(const void *x, int dtype, int64_t m, int64_t k, int64_t ld_x, int use_abs,
                                        void *sparse_out, int64_t ld_sparse, void *mask_out, int64_t ld_mask,
                                        void *stream) {
    if (!x || !mask_out) return SP24_ERR_ARG;
    if (dtype != SP24_F32 && dtype != SP24_F16 && dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (m <= 0 || k <= 0 || m % 32 || k % 64) return SP24_ERR_SHAPE;
    const int sz = dtype_size(dtype);
    if (ld_x < k || (ld_x * sz) % 16 || ld_mask < k || ld_mask % 16) return SP24_ERR_STRIDE;
    if (sparse_out && (ld_sparse < k || (ld_sparse * sz) % 16)) return SP24_ERR_STRIDE;
    if (!aligned16(x) || !aligned16(mask_out) || (sparse_out && !aligned16(sparse_out))) return SP24_ERR_ALIGN;
    if (int rc = check_device()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid((unsigned)((k + 127) / 128), (unsigned)(m / 32));
    uint8_t *mk = static_cast<uint8_t *>(mask_out);
    switch (dtype) {
        case SP24_F32:
            ts_select_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float *>(x), static_cast<float *>(sparse_out), mk,
                                                          k, ld_x, ld_sparse, ld_mask, use_abs);
            break;
        case SP24_F16:
            ts_select_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half *>(x), static_cast<__half *>(sparse_out),
                                                           mk, k, ld_x, ld_sparse, ld_mask, use_abs);
            break;
        default:
            ts_select_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(x),
                                                                  static_cast<__nv_bfloat16 *>(sparse_out), mk, k, ld_x,
                                                                  ld_sparse, ld_mask, use_abs);
    }
    return launch_status();
}

extern "C" int sp24_select_dual_compress(const void *w, int dtype, int64_t m, int64_t k, int64_t ld_w, int select,
                                         void *mask, int64_t ld_mask, void *packed_w, int packed_dtype,
                                         int64_t ld_packed_w, void *meta_w, void *packed_t, int64_t ld_packed_t,
                                         void *meta_t, void *stream) {
    if (!w || !mask || !packed_w || !meta_w || !packed_t || !meta_t) return SP24_ERR_ARG;
    if (dtype != SP24_F32 && dtype != SP24_F16 && dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (packed_dtype != SP24_F16 && packed_dtype != SP24_BF16) return SP24_ERR_DTYPE;
    if (m <= 0 || k <= 0 || m % 64 || k % 64) return SP24_ERR_SHAPE;
    const int sz = dtype_size(dtype);
    if (ld_w < k || (ld_w * sz) % 16 || ld_mask < k || ld_mask % 16) return SP24_ERR_STRIDE;
    if (ld_packed_w < k / 2 || ld_packed_w % 8 || ld_packed_t < k || ld_packed_t % 8) return SP24_ERR_STRIDE;
    if (!aligned16(w) || !aligned16(mask) || !aligned16(packed_w) || !aligned16(meta_w) || !aligned16(packed_t) ||
        !aligned16(meta_t))
        return SP24_ERR_ALIGN;
    if (int rc = check_device()) return rc;
    DualParams P{w, static_cast<uint8_t *>(mask), packed_w, packed_t, static_cast<int16_t *>(meta_w),
                 static_cast<int16_t *>(meta_t), m, k, ld_w, ld_mask, ld_packed_w, ld_packed_t};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case SP24_F32: return dispatch_dual<float>(P, packed_dtype, select, st);
        case SP24_F16: return dispatch_dual<__half>(P, packed_dtype, select, st);
        default: return dispatch_dual<__nv_bfloat16>(P, packed_dtype, select, st);
    }
}
