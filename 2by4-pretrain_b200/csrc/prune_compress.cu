// Dense -> 2:4 compressed conversion: fused prune (magnitude / supplied mask / MVUE) + value
// compaction + metadata packing, for row-major and column-major storage of the logical matrix.
//
// Both kernels are HBM-bound streaming kernels.  Values leave through 16-byte coalesced stores;
// metadata words are first placed in shared memory at their position inside the destination run
// (the reordered layout keeps every aligned group of 32 rows x 2 metadata columns contiguous) and
// then written with 16-byte stores, so no partial sector is ever written.
#include "sp24_common.cuh"

namespace sp24 {
namespace {

struct PcParams {
    const void *dense;
    void *packed;
    void *meta;
    const uint8_t *mask;
    const float *uniforms;
    int64_t m, k, ld_dense, ld_packed, ld_mask, ld_u;
    uint64_t seed, offset;
    const unsigned long long *offset_dev;   // optional device word added to offset at run time
    int16_t *tc;                            // optional metadata copy in tensor-core atom order (16-bit outputs)
    int64_t k_atoms;                        // 128-column atoms per 128-row block
    float *row_sums;                        // optional (column-major only): row_sums[r] += sum over k of dense[r, k]
    int packed_rm;                          // column-major input, 8-bit output: packed is written row-major (m, k/2)
    float out_scale;                        // 8-bit outputs: stored value = value * out_scale (1 = none)
    float soft_scale;                       // soft-threshold mode: kept values are also multiplied by this ...
    int soft_use_scale;                     // ... when this is set (one more rounding in the input type)
};

// internal mode code of the fused soft-threshold + compress entry point (not part of the public enum)
constexpr int PRUNE_SOFT = 4;

template <typename T, int N> __device__ __forceinline__ void load_elems(const T *p, T (&out)[N]) {
    constexpr int PER = (sizeof(T) * N >= 16) ? 16 / sizeof(T) : N;
#pragma unroll
    for (int i = 0; i < N / PER; ++i) {
        Vec<T, PER> v = load_vec<T, PER>(p + i * PER);
#pragma unroll
        for (int j = 0; j < PER; ++j) out[i * PER + j] = v.v[j];
    }
}
template <typename T, int N> __device__ __forceinline__ void store_elems(T *p, const T (&in)[N]) {
    constexpr int PER = (sizeof(T) * N >= 16) ? 16 / sizeof(T) : N;
#pragma unroll
    for (int i = 0; i < N / PER; ++i) {
        Vec<T, PER> v;
#pragma unroll
        for (int j = 0; j < PER; ++j) v.v[j] = in[i * PER + j];
        store_vec<T, PER>(p + i * PER, v);
    }
}

constexpr bool is_mvue(int mode) { return mode == SP24_PRUNE_MVUE || mode == SP24_PRUNE_MVUE_FAST; }
// uniform pairs of the two groups of one Philox block, in the stream of the pruning mode
template <int MODE>
__device__ __forceinline__ void mode_uniform_pairs(uint64_t pair, uint64_t seed, uint64_t offset, float &u0a, float &u1a,
                                                   float &u0b, float &u1b) {
    if constexpr (MODE == SP24_PRUNE_MVUE_FAST) mvue_uniform_pairs_fast(pair, seed, offset, u0a, u1a, u0b, u1b);
    else mvue_uniform_pairs(pair, seed, offset, u0a, u1a, u0b, u1b);
}

// Fast MVUE, after the arithmetic: q[] holds all four quotients, keep the keep mask.  Emits the two stored values
// and returns the 4-bit code.  16-bit outputs: round all four, then one table lookup (keep_lut = words 64..79 of the
// group table, in shared memory) and one byte permute gather the two stored ones.
template <typename TOut>
__device__ __forceinline__ uint32_t emit_fast(const float (&q)[4], uint32_t keep, TOut &o0, TOut &o1, const uint32_t *keep_lut,
                                              float scale = 1.f) {
    if constexpr (sizeof(TOut) == 2) {
        const uint32_t e = keep_lut[keep];
        const uint32_t o = __byte_perm(Elem<TOut>::pack2(q[0], q[1]), Elem<TOut>::pack2(q[2], q[3]), e >> 8);
        const uint16_t lo = (uint16_t)(o & 0xFFFFu), hi = (uint16_t)(o >> 16);
        o0 = *reinterpret_cast<const TOut *>(&lo);
        o1 = *reinterpret_cast<const TOut *>(&hi);
        return e & 0xFu;
    } else {
        // 8-bit outputs: the caller's quantisation scale is applied before the cast (one more float32 rounding)
        const uint32_t nib = encode_nibble(keep);
        o0 = Elem<TOut>::from_f32(__fmul_rn(pick4(nib & 3u, q[0], q[1], q[2], q[3]), scale));
        o1 = Elem<TOut>::from_f32(__fmul_rn(pick4(nib >> 2, q[0], q[1], q[2], q[3]), scale));
        return nib;
    }
}

// One group of four: decide the keep mask, emit the two stored values and the 4-bit code.
// keep_lut: words 64..79 of the group table (indexed by a 4-bit keep mask) in shared memory; only the fast MVUE
// mode with 16-bit outputs reads it.
template <typename TIn, typename TOut, int MODE>
__device__ __forceinline__ uint32_t do_group(const TIn (&in)[4], uint32_t given_mask, float u0, float u1, TOut &o0,
                                             TOut &o1, const uint32_t *keep_lut = nullptr, float scale = 1.f) {
    // `scale` only acts on 8-bit outputs (float8 quantisation); 16-bit outputs ignore it
    constexpr bool SCALED = sizeof(TOut) == 1 && !std::is_same<TOut, int8_t>::value;
    uint32_t keep;
    if constexpr (MODE == SP24_PRUNE_MVUE_FAST) {
        float x[4] = {Elem<TIn>::to_f32(in[0]), Elem<TIn>::to_f32(in[1]), Elem<TIn>::to_f32(in[2]),
                      Elem<TIn>::to_f32(in[3])};
        keep = mvue24_group_fast(x, u0, u1);         // all four quotients in x[]
        return emit_fast<TOut>(x, keep, o0, o1, keep_lut, scale);
    } else if constexpr (MODE == SP24_PRUNE_MVUE) {
        float x[4] = {Elem<TIn>::to_f32(in[0]), Elem<TIn>::to_f32(in[1]), Elem<TIn>::to_f32(in[2]),
                      Elem<TIn>::to_f32(in[3])};
        keep = mvue24_group<false>(x, u0, u1);     // quotients of the two stored positions in x[0], x[1]
        const uint32_t nib = encode_nibble(keep);
        o0 = Elem<TOut>::from_f32(SCALED ? __fmul_rn(x[0], scale) : x[0]);
        o1 = Elem<TOut>::from_f32(SCALED ? __fmul_rn(x[1], scale) : x[1]);
        return nib;
    } else if constexpr (MODE == PRUNE_SOFT) {
        // S-STE: magnitude 2:4 mask; the two kept values move toward zero by the group's second-smallest magnitude
        // (one rounding in the input type), then optionally times the frozen scale (one more rounding in the input
        // type), then the cast to the packed type.  u0 carries the scale, u1 != 0 says whether to apply it.
        const float x0 = Elem<TIn>::to_f32(in[0]), x1 = Elem<TIn>::to_f32(in[1]), x2 = Elem<TIn>::to_f32(in[2]),
                    x3 = Elem<TIn>::to_f32(in[3]);
        keep = magnitude_mask4(x0, x1, x2, x3);
        const float a0 = fabsf(x0), a1 = fabsf(x1), a2 = fabsf(x2), a3 = fabsf(x3);
        const float thr = fminf(fmaxf(fminf(a0, a1), fminf(a2, a3)), fminf(fmaxf(a0, a1), fmaxf(a2, a3)));
        const uint32_t nib = encode_nibble(keep);
        float kv[2] = {pick4(nib & 3u, x0, x1, x2, x3), pick4(nib >> 2, x0, x1, x2, x3)};
        TIn t[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            t[i] = Elem<TIn>::from_f32(kv[i] > 0.f ? __fsub_rn(kv[i], thr) : __fadd_rn(kv[i], thr));
            if (u1 != 0.f) t[i] = Elem<TIn>::from_f32(__fmul_rn(Elem<TIn>::to_f32(t[i]), u0));
        }
        o0 = convert<TOut>(t[0]);
        o1 = convert<TOut>(t[1]);
        return nib;
    } else {
        if constexpr (MODE == SP24_PRUNE_MASK) {
            keep = given_mask;
        } else {
            keep = magnitude_mask4(Elem<TIn>::to_f32(in[0]), Elem<TIn>::to_f32(in[1]), Elem<TIn>::to_f32(in[2]),
                                   Elem<TIn>::to_f32(in[3]));
        }
        const uint32_t nib = encode_nibble(keep);
        if constexpr (SCALED) {
            o0 = Elem<TOut>::from_f32(__fmul_rn(Elem<TIn>::to_f32(pick4(nib & 3u, in[0], in[1], in[2], in[3])), scale));
            o1 = Elem<TOut>::from_f32(__fmul_rn(Elem<TIn>::to_f32(pick4(nib >> 2, in[0], in[1], in[2], in[3])), scale));
        } else {
            o0 = convert<TOut>(pick4(nib & 3u, in[0], in[1], in[2], in[3]));
            o1 = convert<TOut>(pick4(nib >> 2, in[0], in[1], in[2], in[3]));
        }
        return nib;
    }
}

// ---------------------------------------------------------------------------------------------
// Table-driven group processing for 16-bit -> same 16-bit type (magnitude and mask modes).
// Words 0..63: indexed by the six magnitude comparisons x1 | x2<<1 | x3<<2 | x4<<3 | x5<<4 | x6<<5
// (x1 = |a0|>|a1|, x2 = |a0|>|a2|, x3 = |a0|>|a3|, x4 = |a1|>|a2|, x5 = |a1|>|a3|, x6 = |a2|>|a3|);
// words 64..79: indexed by a 4-bit keep mask.  Each word: bits 0..3 the metadata code idx0 | idx1<<2,
// bits 8..23 the byte-permute selector that gathers elements idx0, idx1 from a (lo, hi) register pair.
// ---------------------------------------------------------------------------------------------
struct GroupLut { uint32_t v[80]; };
__host__ __device__ constexpr uint32_t lut_word_for_keep(uint32_t keep) {
    const uint32_t m0 = keep & 1u, m1 = (keep >> 1) & 1u, m2 = (keep >> 2) & 1u;
    const uint32_t bit0 = (m0 ^ 1u) & m1, bit1 = (m0 ^ 1u) & (m1 ^ 1u);
    const uint32_t bit2 = bit1 | (m2 ^ 1u), bit3 = bit0 | (m1 ^ 1u) | m2;
    const uint32_t i0 = bit0 | (bit1 << 1), i1 = bit2 | (bit3 << 1);
    const uint32_t sel = (2 * i0) | ((2 * i0 + 1) << 4) | ((2 * i1) << 8) | ((2 * i1 + 1) << 12);
    return (i0 | (i1 << 2)) | (sel << 8);
}
constexpr GroupLut make_group_lut() {
    GroupLut L{};
    for (uint32_t i = 0; i < 64; ++i) {
        const bool x1 = i & 1, x2 = i & 2, x3 = i & 4, x4 = i & 8, x5 = i & 16, x6 = i & 32;
        const bool m0 = (x2 && x3) || (x1 && x2) || (x1 && x3);
        const bool m1 = (!x1 && x5) || (x4 && x5) || (!x1 && x4);
        const bool m2 = (!x2 && !x4) || (!x2 && x6) || (!x4 && x6);
        const bool m3 = (!x3 && !x5) || (!x3 && !x6) || (!x5 && !x6);
        L.v[i] = lut_word_for_keep((uint32_t)m0 | ((uint32_t)m1 << 1) | ((uint32_t)m2 << 2) | ((uint32_t)m3 << 3));
    }
    for (uint32_t k = 0; k < 16; ++k) L.v[64 + k] = lut_word_for_keep(k);
    return L;
}
__constant__ GroupLut kGroupLut = make_group_lut();

template <typename T> struct Packed16;
template <> struct Packed16<__half> {
    __device__ static uint32_t gt_mask(uint32_t a, uint32_t b) {
        return __hgt2_mask(*reinterpret_cast<const __half2 *>(&a), *reinterpret_cast<const __half2 *>(&b));
    }
};
template <> struct Packed16<__nv_bfloat16> {
    __device__ static uint32_t gt_mask(uint32_t a, uint32_t b) {
        return __hgt2_mask(*reinterpret_cast<const __nv_bfloat162 *>(&a), *reinterpret_cast<const __nv_bfloat162 *>(&b));
    }
};

// lo = (x0, x1), hi = (x2, x3) as packed 16-bit values.  Returns the table word of the magnitude rule.
template <typename T> __device__ __forceinline__ uint32_t mse_lookup(uint32_t lo, uint32_t hi, const uint32_t *lut) {
    const uint32_t a = lo & 0x7FFF7FFFu, b = hi & 0x7FFF7FFFu;          // |x0|,|x1| and |x2|,|x3|
    const uint32_t c1 = Packed16<T>::gt_mask(a, b);                       // x2 (low half), x5 (high half)
    const uint32_t c2 = Packed16<T>::gt_mask(a, __byte_perm(b, b, 0x1032));  // x3, x4
    const uint32_t c3 = Packed16<T>::gt_mask(__byte_perm(a, b, 0x5410), __byte_perm(a, b, 0x7632));  // x1, x6
    const uint32_t t = (c3 & 0x00200001u) | (c1 & 0x00100002u) | (c2 & 0x00080004u);
    return lut[(t | (t >> 16)) & 0x3Fu];
}

// ---------------------------------------------------------------------------------------------
// row-major storage: groups of four run along the contiguous axis.
// Tile = 32 rows x 32 metadata columns; 8 warps, lane = metadata column, warp w owns rows 4w..4w+3.
// ---------------------------------------------------------------------------------------------
template <typename TIn, typename TOut, int MODE, bool HAS_U>
__global__ void __launch_bounds__(256, is_mvue(MODE) ? 3 : 1) pc_row_kernel(PcParams P) {
    const uint64_t rng_offset = P.offset + (P.offset_dev ? *P.offset_dev : 0ull);
    constexpr int CH = sizeof(TOut) == 2 ? 16 : 32;  // dense elements per metadata word
    constexpr int MB = sizeof(TOut) == 2 ? 2 : 4;    // bytes per metadata word
    constexpr int GROUP = MB == 2 ? 32 : 16;
    using MetaT = typename VecBytes<MB>::type;
    // rows in flight per thread; MVUE is arithmetic-bound, so it trades memory-level parallelism for
    // fewer registers (more resident warps)
    constexpr int RPI = (is_mvue(MODE) || CH * sizeof(TIn) >= 128) ? 1 : (CH * sizeof(TIn) >= 64 ? 2 : 4);

    __shared__ __align__(16) MetaT smeta[16][64];
    constexpr bool PACKED = !is_mvue(MODE) && MODE != PRUNE_SOFT && std::is_same<TIn, TOut>::value && sizeof(TIn) == 2;
    constexpr bool KEEP_LUT = MODE == SP24_PRUNE_MVUE_FAST && sizeof(TOut) == 2;   // words 64..79 only
    __shared__ uint32_t glut[PACKED ? 80 : (KEEP_LUT ? 16 : 1)];
    if constexpr (PACKED) {
        if (threadIdx.x < 80) glut[threadIdx.x] = kGroupLut.v[threadIdx.x];
        __syncthreads();
    }
    if constexpr (KEEP_LUT) {
        if (threadIdx.x < 16) glut[threadIdx.x] = kGroupLut.v[64 + threadIdx.x];
        __syncthreads();
    }

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t ncols = P.k / CH;
    const int64_t c = (int64_t)blockIdx.x * 32 + lane;
    const int64_t r0 = (int64_t)blockIdx.y * 32;
    const TIn *dense = static_cast<const TIn *>(P.dense);
    TOut *packed = static_cast<TOut *>(P.packed);

    if (c < ncols) {
#pragma unroll(is_mvue(MODE) ? 1 : 4)
        for (int it = 0; it < 4 / RPI; ++it) {
            TIn in[RPI][CH];
            uint8_t mk[RPI][CH];
#pragma unroll
            for (int j = 0; j < RPI; ++j) {
                const int64_t r = r0 + warp * 4 + it * RPI + j;
                load_elems<TIn, CH>(dense + r * P.ld_dense + c * CH, in[j]);
                if constexpr (MODE == SP24_PRUNE_MASK) load_elems<uint8_t, CH>(P.mask + r * P.ld_mask + c * CH, mk[j]);
            }
#pragma unroll
            for (int j = 0; j < RPI; ++j) {
                const int rr = warp * 4 + it * RPI + j;
                const int64_t r = r0 + rr;
                TOut out[CH / 2];
                uint32_t word = 0;
                if constexpr (PACKED) {
                    // one table lookup and one byte permute per group of four
                    const uint32_t *raw = reinterpret_cast<const uint32_t *>(&in[j][0]);
                    uint32_t *o32 = reinterpret_cast<uint32_t *>(&out[0]);
#pragma unroll
                    for (int g = 0; g < CH / 4; ++g) {
                        uint32_t e;
                        if constexpr (MODE == SP24_PRUNE_MASK) {
                            const uint32_t mw = *reinterpret_cast<const uint32_t *>(&mk[j][4 * g]);
                            e = glut[64 + (((__vcmpne4(mw, 0u) & 0x01010101u) * 0x01020408u) >> 24)];
                        } else {
                            e = mse_lookup<TIn>(raw[2 * g], raw[2 * g + 1], glut);
                        }
                        o32[g] = __byte_perm(raw[2 * g], raw[2 * g + 1], e >> 8);
                        word |= (e & 0xFu) << (4 * g);
                    }
                } else
#pragma unroll
                for (int g2 = 0; g2 < CH / 8; ++g2) {
                    float u[4] = {0.f, 0.f, 0.f, 0.f};
                    if constexpr (MODE == PRUNE_SOFT) { u[0] = u[2] = P.soft_scale; u[1] = u[3] = P.soft_use_scale ? 1.f : 0.f; }
                    if constexpr (is_mvue(MODE)) {
                        if constexpr (HAS_U) {
                            const float *up = P.uniforms + r * P.ld_u + c * CH + g2 * 8;
                            const float2 ua = *reinterpret_cast<const float2 *>(up);
                            const float2 ub = *reinterpret_cast<const float2 *>(up + 4);
                            u[0] = ua.x; u[1] = ua.y; u[2] = ub.x; u[3] = ub.y;
                        } else {
                            const uint64_t gi = (uint64_t)r * (uint64_t)(P.k / 4) + (uint64_t)(c * (CH / 4) + g2 * 2);
                            mode_uniform_pairs<MODE>(gi >> 1, P.seed, rng_offset, u[0], u[1], u[2], u[3]);
                        }
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int g = g2 * 2 + h;
                        const TIn grp[4] = {in[j][4 * g], in[j][4 * g + 1], in[j][4 * g + 2], in[j][4 * g + 3]};
                        uint32_t given = 0;
                        if constexpr (MODE == SP24_PRUNE_MASK) {
                            given = (mk[j][4 * g] != 0) | ((mk[j][4 * g + 1] != 0) << 1) | ((mk[j][4 * g + 2] != 0) << 2) |
                                    ((mk[j][4 * g + 3] != 0) << 3);
                        }
                        const uint32_t nib =
                            do_group<TIn, TOut, MODE>(grp, given, u[2 * h], u[2 * h + 1], out[2 * g], out[2 * g + 1], glut, P.out_scale);
                        word |= nib << (4 * g);
                    }
                }
                store_elems<TOut, CH / 2>(packed + r * P.ld_packed + c * (CH / 2), out);
                smeta[lane >> 1][(rr / GROUP) * 2 * GROUP + meta_run_pos<MB>(rr % GROUP, lane & 1)] = (MetaT)word;
            }
        }
    }
    __syncthreads();
    // 16 column pairs x 64 words, written as 16-byte pieces
    constexpr int PIECES = 64 * MB / 16;
    for (int i = threadIdx.x; i < 16 * PIECES; i += 256) {
        const int pair = i / PIECES, piece = i % PIECES;
        const int64_t cp = (int64_t)blockIdx.x * 16 + pair;
        if (cp * 2 < ncols) {
            char *dst = static_cast<char *>(P.meta) + (cp * 2 * P.m + 2 * r0) * MB + piece * 16;
            *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(
                reinterpret_cast<const char *>(&smeta[pair][0]) + piece * 16);
        }
    }
    if constexpr (MB == 2) {
        if (P.tc && threadIdx.x < 128) {
            // Second copy in tensor-core order, gathered from the staged runs: the tile's 32 rows x 32 word columns
            // are 32 whole 16-byte lines in each of four atoms.  Line L holds rows 16*(L/16) + 8*h + L%8 (h = 0, 1) of
            // word columns 2*q + (L/8)%2 (q = 0..3) at int16 slot 2*q + h.
            const int atom = threadIdx.x >> 5, L = threadIdx.x & 31, par = (L >> 3) & 1;
            const int64_t atom_col = (int64_t)blockIdx.x * 4 + atom;
            if (atom_col < P.k_atoms) {
                uint32_t o[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int wc = atom * 8 + 2 * q + par;                  // word column inside the tile
                    uint32_t lo = 0, hi = 0;
                    if ((int64_t)blockIdx.x * 32 + wc < ncols) {
                        lo = (uint16_t)smeta[wc >> 1][meta_run_pos<MB>(16 * (L >> 4) + (L & 7), wc & 1)];
                        hi = (uint16_t)smeta[wc >> 1][meta_run_pos<MB>(16 * (L >> 4) + 8 + (L & 7), wc & 1)];
                    }
                    o[q] = lo | (hi << 16);
                }
                const int64_t off = ((r0 >> 7) * P.k_atoms + atom_col) * 2048 + ((r0 & 127) + L) * 16;
                if (off + 16 <= (P.m >> 7) * P.k_atoms * 2048)   // every store is checked against the buffer size
                    *reinterpret_cast<uint4 *>(reinterpret_cast<char *>(P.tc) + off) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// column-major storage: element (r, c) at c*ld + r, groups of four run along the strided axis.
// Everything is element-wise across r, so loads and stores are naturally coalesced along r.
// Thread = V consecutive rows x one metadata column; warp = 32*V rows; 8 warps = 8 metadata columns.
// ---------------------------------------------------------------------------------------------
template <typename TIn> struct ColVec {
    static constexpr int wide = sizeof(TIn) == 1 ? 8 : 16 / sizeof(TIn);   // streaming modes: 16-byte (8 for int8) loads
    // Exact MVUE is bound by instruction issue, not by load width: one row per thread makes blocks of 32 rows, which
    // balances the SMs better on short matrices and is never slower on long ones.
    static constexpr int narrow = 1;
    // Fast MVUE has a third of the arithmetic, so its loads and stores weigh more: four rows per thread (8-byte
    // accesses for 16-bit inputs) is the fastest from 768 x 8192 to 4096 x 8192 (one / two rows: +7 % / +3 %).
    static constexpr int fast = 4;
};

// resident blocks per SM the register budget is set for
constexpr int col_min_blocks(int mode) { return mode == SP24_PRUNE_MVUE_FAST ? 3 : (mode == SP24_PRUNE_MVUE ? 4 : 1); }

template <typename TIn, typename TOut, int MODE, bool HAS_U, int V>
__global__ void __launch_bounds__(256, col_min_blocks(MODE)) pc_col_kernel(PcParams P) {
    const uint64_t rng_offset = P.offset + (P.offset_dev ? *P.offset_dev : 0ull);
    constexpr int CH = sizeof(TOut) == 2 ? 16 : 32;
    constexpr int MB = sizeof(TOut) == 2 ? 2 : 4;
    constexpr int GROUP = MB == 2 ? 32 : 16;
    constexpr int RT = 32 * V;  // rows per block
    using MetaT = typename VecBytes<MB>::type;

    __shared__ __align__(16) MetaT smeta[4][2 * RT];
    // tensor-core order: line L = 16*(r/16) + 8*(c%2) + r%8 of 16 bytes, int16 slot 2*((c/2)%4) + (r/8)%2; the block's
    // RT rows x 8 word columns fill RT whole lines of one atom per 128-row block
    __shared__ __align__(16) uint16_t stc[MB == 2 ? RT * 8 : 8];
    __shared__ float ssum[8][RT];           // per-warp partial row sums (only used when row sums are asked for)
    constexpr bool KEEP_LUT = MODE == SP24_PRUNE_MVUE_FAST && sizeof(TOut) == 2;
    __shared__ uint32_t glut[KEEP_LUT ? 16 : 1];
    if constexpr (KEEP_LUT) {
        if (threadIdx.x < 16) glut[threadIdx.x] = kGroupLut.v[64 + threadIdx.x];
        __syncthreads();
    }

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t ncols = P.k / CH;
    const int64_t r0 = (int64_t)blockIdx.x * RT;
    const int64_t r = r0 + lane * V;
    const int64_t c = (int64_t)blockIdx.y * 8 + warp;
    TOut *packed = static_cast<TOut *>(P.packed);

    if (r < P.m && c < ncols) {
        uint32_t word[V];
        float rsum[V];
#pragma unroll
        for (int v = 0; v < V; ++v) { word[v] = 0; rsum[v] = 0.f; }
        // one running pointer per array: the eight storage rows of a step are ld apart
        const TIn *src = static_cast<const TIn *>(P.dense) + (c * CH) * P.ld_dense + r;
        const uint8_t *msrc = MODE == SP24_PRUNE_MASK ? P.mask + (c * CH) * P.ld_mask + r : nullptr;
        TOut *dst = packed + (c * (CH / 2)) * P.ld_packed + r;
        // 8-bit outputs can also leave row-major (the K-major operand order of the 8-bit sparse GEMM): a thread's
        // 32 logical columns are 16 contiguous packed bytes of its row
        constexpr bool CAN_RM = sizeof(TOut) == 1;
        TOut orow[CAN_RM ? V : 1][CAN_RM ? CH / 2 : 1];
        // a step = 8 consecutive storage rows = two groups of four per logical row = one Philox block
#pragma unroll
        for (int step = 0; step < CH / 8; ++step) {
            Vec<TIn, V> in[8];
            Vec<uint8_t, V> mk[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                in[j] = load_vec<TIn, V>(src + j * P.ld_dense);
                if constexpr (MODE == SP24_PRUNE_MASK) mk[j] = load_vec<uint8_t, V>(msrc + j * P.ld_mask);
            }
            src += 8 * P.ld_dense;
            if constexpr (MODE == SP24_PRUNE_MASK) msrc += 8 * P.ld_mask;
            if (P.row_sums) {   // sums of the unpruned values, fp32
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    float a = 0.f;
#pragma unroll
                    for (int j = 0; j < 8; ++j) a += Elem<TIn>::to_f32(in[j].v[v]);
                    rsum[v] += a;
                }
            }
            float u[V][4];
            if constexpr (is_mvue(MODE)) {
                const int64_t gcol = c * (CH / 4) + step * 2;  // first of the two groups
                if constexpr (HAS_U) {
                    float t0[V], t1[V], t2[V], t3[V];
                    load_elems<float, V>(P.uniforms + (gcol * 4 + 0) * P.ld_u + r, t0);
                    load_elems<float, V>(P.uniforms + (gcol * 4 + 1) * P.ld_u + r, t1);
                    load_elems<float, V>(P.uniforms + (gcol * 4 + 4) * P.ld_u + r, t2);
                    load_elems<float, V>(P.uniforms + (gcol * 4 + 5) * P.ld_u + r, t3);
#pragma unroll
                    for (int v = 0; v < V; ++v) { u[v][0] = t0[v]; u[v][1] = t1[v]; u[v][2] = t2[v]; u[v][3] = t3[v]; }
                } else {
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        const uint64_t gi = (uint64_t)(r + v) * (uint64_t)(P.k / 4) + (uint64_t)gcol;
                        mode_uniform_pairs<MODE>(gi >> 1, P.seed, rng_offset, u[v][0], u[v][1], u[v][2], u[v][3]);
                    }
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                Vec<TOut, V> o0, o1;
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    const TIn grp[4] = {in[4 * h].v[v], in[4 * h + 1].v[v], in[4 * h + 2].v[v], in[4 * h + 3].v[v]};
                    uint32_t given = 0;
                    if constexpr (MODE == SP24_PRUNE_MASK) {
                        given = (mk[4 * h].v[v] != 0) | ((mk[4 * h + 1].v[v] != 0) << 1) | ((mk[4 * h + 2].v[v] != 0) << 2) |
                                ((mk[4 * h + 3].v[v] != 0) << 3);
                    }
                    float ua = 0.f, ub = 0.f;
                    if constexpr (is_mvue(MODE)) { ua = u[v][2 * h]; ub = u[v][2 * h + 1]; }
                    if constexpr (MODE == PRUNE_SOFT) { ua = P.soft_scale; ub = P.soft_use_scale ? 1.f : 0.f; }
                    const uint32_t nib = do_group<TIn, TOut, MODE>(grp, given, ua, ub, o0.v[v], o1.v[v], glut, P.out_scale);
                    word[v] |= nib << (4 * (step * 2 + h));
                    if constexpr (CAN_RM) {
                        orow[v][(step * 2 + h) * 2] = o0.v[v];
                        orow[v][(step * 2 + h) * 2 + 1] = o1.v[v];
                    }
                }
                if (!CAN_RM || !P.packed_rm) {
                    store_vec<TOut, V>(dst, o0);
                    store_vec<TOut, V>(dst + P.ld_packed, o1);
                    dst += 2 * P.ld_packed;
                }
            }
        }
        if constexpr (CAN_RM) {
            if (P.packed_rm) {
#pragma unroll
                for (int v = 0; v < V; ++v) store_elems<TOut, CH / 2>(packed + (r + v) * P.ld_packed + c * (CH / 2), orow[v]);
            }
        }
        if (P.row_sums) {
#pragma unroll
            for (int v = 0; v < V; ++v) ssum[warp][lane * V + v] = rsum[v];
        }
#pragma unroll
        for (int v = 0; v < V; ++v) {
            const int rr = lane * V + v;
            smeta[warp >> 1][(rr / GROUP) * 2 * GROUP + meta_run_pos<MB>(rr % GROUP, warp & 1)] = (MetaT)word[v];
            if constexpr (MB == 2)
                if (P.tc) stc[8 * (16 * (rr >> 4) + 8 * (warp & 1) + (rr & 7)) + 2 * (warp >> 1) + ((rr >> 3) & 1)] = (uint16_t)word[v];
        }
    } else {
        if (P.row_sums) {
#pragma unroll
            for (int v = 0; v < V; ++v) ssum[warp][lane * V + v] = 0.f;
        }
        if constexpr (MB == 2) {
            // word columns past the matrix (K not a multiple of 128): zeros, the GEMM multiplies them by zero-filled operands
            if (P.tc && r < P.m) {
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    const int rr = lane * V + v;
                    stc[8 * (16 * (rr >> 4) + 8 * (warp & 1) + (rr & 7)) + 2 * (warp >> 1) + ((rr >> 3) & 1)] = 0;
                }
            }
        }
    }
    __syncthreads();
    if (P.row_sums) {
        // the eight warps hold eight K ranges of the same rows: one reduction per row and block
        for (int t = threadIdx.x; t < RT; t += 256) {
            if (r0 + t < P.m) {
                float a = 0.f;
#pragma unroll
                for (int w = 0; w < 8; ++w) a += ssum[w][t];
                atomicAdd(P.row_sums + r0 + t, a);
            }
        }
    }
    const int64_t rows_here = (P.m - r0 < RT) ? (P.m - r0) : RT;
    const int pieces = (int)(rows_here * 2 * MB / 16);
    for (int i = threadIdx.x; i < 4 * (2 * RT * MB / 16); i += 256) {
        const int pair = i / (2 * RT * MB / 16), piece = i % (2 * RT * MB / 16);
        const int64_t cp = (int64_t)blockIdx.y * 4 + pair;
        if (piece < pieces && cp * 2 < ncols) {
            char *dstm = static_cast<char *>(P.meta) + (cp * 2 * P.m + 2 * r0) * MB + piece * 16;
            *reinterpret_cast<uint4 *>(dstm) = *reinterpret_cast<const uint4 *>(
                reinterpret_cast<const char *>(&smeta[pair][0]) + piece * 16);
        }
    }
    if constexpr (MB == 2) {
        if (P.tc) {
            for (int pline = threadIdx.x; pline < RT; pline += 256) {
                if (pline < rows_here) {
                    const int64_t gr = r0 + pline;   // line index inside the 128-row block = row index of its first writer
                    const int64_t off = ((gr >> 7) * P.k_atoms + blockIdx.y) * 2048 + (gr & 127) * 16;
                    if (off + 16 <= (P.m >> 7) * P.k_atoms * 2048)   // every store is checked against the buffer size
                        *reinterpret_cast<uint4 *>(reinterpret_cast<char *>(P.tc) + off) =
                            *reinterpret_cast<const uint4 *>(reinterpret_cast<const char *>(stc) + pline * 16);
                }
            }
        }
    }
}

template <typename TIn, typename TOut, int MODE, bool HAS_U>
int launch(const PcParams &P, int col_major, cudaStream_t st) {
    constexpr int CH = sizeof(TOut) == 2 ? 16 : 32;
    if (!col_major) {
        dim3 grid((unsigned)((P.k / CH + 31) / 32), (unsigned)(P.m / 32));
        pc_row_kernel<TIn, TOut, MODE, HAS_U><<<grid, 256, 0, st>>>(P);
    } else {
        constexpr int V = MODE == SP24_PRUNE_MVUE_FAST ? ColVec<TIn>::fast : (MODE == SP24_PRUNE_MVUE ? ColVec<TIn>::narrow : ColVec<TIn>::wide);
        constexpr int RT = 32 * V;
        dim3 grid((unsigned)((P.m + RT - 1) / RT), (unsigned)((P.k / CH + 7) / 8));
        pc_col_kernel<TIn, TOut, MODE, HAS_U, V><<<grid, 256, 0, st>>>(P);
    }
    return launch_status();
}

template <typename TIn, typename TOut> int dispatch_mode(const PcParams &P, int mode, int col_major, cudaStream_t st) {
    switch (mode) {
        case SP24_PRUNE_MSE: return launch<TIn, TOut, SP24_PRUNE_MSE, false>(P, col_major, st);
        case SP24_PRUNE_MASK: return launch<TIn, TOut, SP24_PRUNE_MASK, false>(P, col_major, st);
        case SP24_PRUNE_MVUE:
            if constexpr (std::is_same<TIn, int8_t>::value) {
                return SP24_ERR_DTYPE;
            } else {
                return P.uniforms ? launch<TIn, TOut, SP24_PRUNE_MVUE, true>(P, col_major, st)
                                  : launch<TIn, TOut, SP24_PRUNE_MVUE, false>(P, col_major, st);
            }
        case SP24_PRUNE_MVUE_FAST:
            if constexpr (std::is_same<TIn, int8_t>::value) return SP24_ERR_DTYPE;
            else return launch<TIn, TOut, SP24_PRUNE_MVUE_FAST, false>(P, col_major, st);
        case PRUNE_SOFT:
            if constexpr (std::is_same<TIn, int8_t>::value || sizeof(TOut) != 2) return SP24_ERR_DTYPE;
            else return launch<TIn, TOut, PRUNE_SOFT, false>(P, col_major, st);
        default: return SP24_ERR_ARG;
    }
}

template <typename TIn> int dispatch_out(const PcParams &P, int packed_dtype, int mode, int col_major, cudaStream_t st) {
    switch (packed_dtype) {
        case SP24_F16: return dispatch_mode<TIn, __half>(P, mode, col_major, st);
        case SP24_BF16: return dispatch_mode<TIn, __nv_bfloat16>(P, mode, col_major, st);
        case SP24_E4M3: return dispatch_mode<TIn, e4m3_t>(P, mode, col_major, st);
        case SP24_E5M2: return dispatch_mode<TIn, e5m2_t>(P, mode, col_major, st);
        default: return SP24_ERR_DTYPE;
    }
}

}  // namespace
}  // namespace sp24

static int prune_compress_impl(const void *dense, int dense_dtype, int64_t m, int64_t k, int64_t ld_dense,
                               int col_major, void *packed, int packed_dtype, int64_t ld_packed, void *meta,
                               int mode, const void *mask, int64_t ld_mask, const float *uniforms,
                               int64_t ld_uniforms, uint64_t seed, uint64_t offset, const uint64_t *offset_dev,
                               void *e_tc, float *row_sums, void *stream, int packed_rm = 0, float out_scale = 1.f,
                               int soft_use_scale = 0, float soft_scale = 1.f) {
    using namespace sp24;
    if (!dense || !packed || !meta) return SP24_ERR_ARG;
    const int so = dtype_size(packed_dtype), si = dtype_size(dense_dtype);
    if (so == 0 || si == 0 || packed_dtype == SP24_F32) return SP24_ERR_DTYPE;
    if (dense_dtype == SP24_E4M3 || dense_dtype == SP24_E5M2) return SP24_ERR_DTYPE;
    if ((dense_dtype == SP24_I8) != (packed_dtype == SP24_I8)) return SP24_ERR_DTYPE;
    const int64_t kmult = so == 2 ? 64 : 128;
    if (m <= 0 || k <= 0 || m % 32 || k % kmult) return SP24_ERR_SHAPE;
    if (mode == SP24_PRUNE_MASK && !mask) return SP24_ERR_ARG;
    if (mode != SP24_PRUNE_MASK && mask) return SP24_ERR_ARG;
    if (mode != SP24_PRUNE_MVUE && uniforms) return SP24_ERR_ARG;
    if (mode < SP24_PRUNE_MSE || mode > PRUNE_SOFT) return SP24_ERR_ARG;
    if (packed_rm && (!col_major || so != 1)) return SP24_ERR_ARG;
    if (!(out_scale > 0.f) || (out_scale != 1.f && (so != 1 || packed_dtype == SP24_I8))) return SP24_ERR_ARG;
    const int64_t inner = col_major ? m : k, inner_p = (col_major && !packed_rm) ? m : k / 2;
    if (ld_dense < inner || (ld_dense * si) % 16) return SP24_ERR_STRIDE;
    if (ld_packed < inner_p || (ld_packed * so) % 16) return SP24_ERR_STRIDE;
    if (mask && (ld_mask < inner || ld_mask % 16)) return SP24_ERR_STRIDE;
    if (uniforms && (ld_uniforms < inner || ld_uniforms % 4)) return SP24_ERR_STRIDE;
    if (!aligned16(dense) || !aligned16(packed) || !aligned16(meta) || (mask && !aligned16(mask)) ||
        (uniforms && !aligned16(uniforms)))
        return SP24_ERR_ALIGN;
    if (e_tc && (so != 2 || m % 128 || !aligned16(e_tc))) return SP24_ERR_ARG;
    if (row_sums && (!col_major || (reinterpret_cast<uintptr_t>(row_sums) & 3u))) return SP24_ERR_ARG;
    if (int rc = check_device()) return rc;
    PcParams P{dense, packed, meta, static_cast<const uint8_t *>(mask), uniforms, m, k, ld_dense, ld_packed, ld_mask,
               ld_uniforms, seed, offset, reinterpret_cast<const unsigned long long *>(offset_dev),
               static_cast<int16_t *>(e_tc), (k + 127) / 128, row_sums, packed_rm, out_scale, soft_scale, soft_use_scale};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dense_dtype) {
        case SP24_F32: return dispatch_out<float>(P, packed_dtype, mode, col_major, st);
        case SP24_F16: return dispatch_out<__half>(P, packed_dtype, mode, col_major, st);
        case SP24_BF16: return dispatch_out<__nv_bfloat16>(P, packed_dtype, mode, col_major, st);
        case SP24_I8: return dispatch_mode<int8_t, int8_t>(P, mode, col_major, st);
        default: return SP24_ERR_DTYPE;
    }
}

extern "C" int sp24_prune_compress(const void *dense, int dense_dtype, int64_t m, int64_t k, int64_t ld_dense,
                                   int col_major, void *packed, int packed_dtype, int64_t ld_packed, void *meta,
                                   int mode, const void *mask, int64_t ld_mask, const float *uniforms,
                                   int64_t ld_uniforms, uint64_t seed, uint64_t offset, void *stream) {
    if (mode > SP24_PRUNE_MVUE_FAST) return SP24_ERR_ARG;
    return prune_compress_impl(dense, dense_dtype, m, k, ld_dense, col_major, packed, packed_dtype, ld_packed, meta, mode,
                               mask, ld_mask, uniforms, ld_uniforms, seed, offset, nullptr, nullptr, nullptr, stream);
}

// Same conversion with three optional extras (each may be NULL).
// offset_dev: the Philox offset becomes `offset` plus the 64-bit word at `offset_dev` (device memory), read when the
//   kernel runs.  A launch recorded once (a CUDA graph) then draws fresh uniforms on every replay if the caller
//   bumps that word between replays.
// e_tc: a second copy of the metadata in the order the sparse GEMM reads (sp24_meta_tc_bytes(m, k) bytes), so that
//   no conversion launch is needed before sp24_spmm.  16-bit outputs only, m % 128 == 0.
// row_sums: m floats; row_sums[r] += sum over k of dense[r, k] (the values before pruning, fp32 partial sums added
//   with atomics: the caller zeroes the array or passes a gradient buffer).  Column-major storage only: for dY^T this
//   is the bias gradient, taken from the pass that reads dY anyway.
extern "C" int sp24_prune_compress_ex(const void *dense, int dense_dtype, int64_t m, int64_t k, int64_t ld_dense,
                                      int col_major, void *packed, int packed_dtype, int64_t ld_packed, void *meta,
                                      int mode, const void *mask, int64_t ld_mask, const float *uniforms,
                                      int64_t ld_uniforms, uint64_t seed, uint64_t offset, const uint64_t *offset_dev,
                                      void *e_tc, float *row_sums, void *stream) {
    if (offset_dev && (reinterpret_cast<uintptr_t>(offset_dev) & 7u)) return SP24_ERR_ARG;
    if (mode > SP24_PRUNE_MVUE_FAST) return SP24_ERR_ARG;
    return prune_compress_impl(dense, dense_dtype, m, k, ld_dense, col_major, packed, packed_dtype, ld_packed, meta, mode,
                               mask, ld_mask, uniforms, ld_uniforms, seed, offset, offset_dev, e_tc, row_sums, stream);
}

// Float8 quantising form of the conversion: packed is ALWAYS row-major (m, k/2), the K-major operand order the 8-bit
// sparse GEMM requires, whatever the storage order of dense (col_major = 1: a transposed view such as W.T of a
// row-major weight or dY.T of a row-major gradient, converted without a transpose pass).  Stored values are
// value * out_scale rounded to the float8 type (the caller's per-tensor quantisation scale; 1 for none).  mask follows
// the storage order of dense.  Metadata: m*k/32 int32 in the reference's reordered layout, as for any 8-bit output.
extern "C" int sp24_prune_compress_q8(const void *dense, int dense_dtype, int64_t m, int64_t k, int64_t ld_dense, int col_major,
                                      void *packed, int packed_dtype, int64_t ld_packed, void *meta, int mode,
                                      const void *mask, int64_t ld_mask, float out_scale, uint64_t seed, uint64_t offset,
                                      void *stream) {
    if (packed_dtype != SP24_E4M3 && packed_dtype != SP24_E5M2) return SP24_ERR_DTYPE;
    if (mode > SP24_PRUNE_MVUE_FAST) return SP24_ERR_ARG;
    return prune_compress_impl(dense, dense_dtype, m, k, ld_dense, col_major, packed, packed_dtype, ld_packed, meta, mode, mask,
                               ld_mask, nullptr, 0, seed, offset, nullptr, nullptr, nullptr, stream, col_major ? 1 : 0,
                               out_scale);
}

// S-STE forward in one pass: magnitude 2:4 mask, soft threshold of the kept values (one rounding in the input type),
// optional frozen scale (one more rounding in the input type), cast to the packed 16-bit type, metadata - what
// sp24_soft_threshold24 followed by a cast and sp24_prune_compress (mask mode) produce in three passes over W.
// e_tc (optional): the metadata also in the order sp24_spmm reads (m % 128 == 0).
extern "C" int sp24_soft_threshold24_compress(const void *dense, int dense_dtype, int64_t m, int64_t k, int64_t ld_dense,
                                              int col_major, void *packed, int packed_dtype, int64_t ld_packed, void *meta,
                                              int use_scale, float scale, void *e_tc, void *stream) {
    if (packed_dtype != SP24_F16 && packed_dtype != SP24_BF16) return SP24_ERR_DTYPE;
    return prune_compress_impl(dense, dense_dtype, m, k, ld_dense, col_major, packed, packed_dtype, ld_packed, meta,
                               sp24::PRUNE_SOFT, nullptr, 0, nullptr, 0, 0, 0, nullptr, e_tc, nullptr, stream, 0, 1.f,
                               use_scale ? 1 : 0, scale);
}
